"""CPU oracle for the DeepBind hot path -- TEST INFRASTRUCTURE ONLY.

ctypes front end for ``libdeepbind_oracle.so`` (the plain-C restatement in
``deepbind_oracle.c``) plus NumPy restatements of the small dense layers, the
losses and the composite networks.  Nothing in the product package imports this
module; the tests, the smoke check and the benchmark's CPU-baseline legs do.

Parity status: the reference holds no golden vectors for this path.  The oracle
is pinned by the reference's own code run beside it: its CUDA kernels and launchers
(scan, pooling, update, masks, dropout, block-diagonal products, smat's element-wise
kernels under the layer math) compiled from its sources for the test GPU
(oracle/build_ref.sh, oracle/ref_shim.cu; tests/test_gpu_ref_kernels.py,
tests/test_gpu_ref_deepity.py, tests/test_gpu_ref_layers.py), and the Python it uses
for ordinal encoding, reverse complement, batch assembly and strand selection, executed
where it lies into a committed fixture (tests/golden/make_ref_util.py,
tests/test_ref_util_tables.py); plus hand-derived known-answer cases
(tests/test_oracle_kat.py).  Not pinned by reference code: column sums of the bias
gradient (the reference's reduction order is its own) and random initialisation.

All arrays are C-contiguous NumPy arrays; layouts follow the reference:
W [4m, nf] (tap-major, channel, filter fastest), X uint8 [npos], regions
uint32 [nregion, 2|3], Z [npos, nf], pooled [nregion, nf|2nf].
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

PT = {"max": 0, "avg": 1, "sum": 2, "all": 3}


def build(force=False):
    so = os.path.join(_HERE, "libdeepbind_oracle.so")
    src = os.path.join(_HERE, "deepbind_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libdeepbind_oracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _suf(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError("oracle supports float32/float64 only")


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


u32 = ctypes.c_uint32


# --------------------------------------------------------------------- scan
def corr1ord(W, X, Z=None):
    """kangaroo_smat.corr1ord: Z is zero-filled here as corr1ord.py:101 does."""
    W = _c(W); X = _c(X, np.uint8).ravel()
    m, nf = W.shape[0] // 4, W.shape[1]
    if Z is None:
        Z = np.zeros((X.size, nf), W.dtype)
    getattr(lib(), "orc_corr1ord_" + _suf(W.dtype))(_p(W), u32(m), u32(nf), _p(X), u32(X.size), _p(Z))
    return Z


def corr1ord_bprop_W(dW, X, dZ):
    X = _c(X, np.uint8).ravel(); dZ = _c(dZ)
    m, nf = dW.shape[0] // 4, dW.shape[1]
    getattr(lib(), "orc_corr1ord_bprop_W_" + _suf(dW.dtype))(_p(dW), u32(m), u32(nf), _p(X), u32(X.size), _p(dZ))
    return dW


def corr1ord_bprop_X(dX, W, dZ):
    W = _c(W); dZ = _c(dZ)
    m, nf = W.shape[0] // 4, W.shape[1]
    getattr(lib(), "orc_corr1ord_bprop_X_" + _suf(W.dtype))(_p(dX), u32(dX.shape[0]), _p(W), u32(m), u32(nf), _p(dZ))
    return dX


# ------------------------------------------------------------------ pooling
def poolrgn(U, R, ptype, want_argmax=False):
    U = _c(U); R = _c(R, np.uint32)
    nf = U.shape[1]; nreg = R.shape[0]
    P = np.empty((nreg, nf * (2 if ptype == "all" else 1)), U.dtype)
    A = np.empty((nreg, nf), np.uint32) if (want_argmax and ptype in ("max", "all")) else None
    getattr(lib(), "orc_poolrgn_" + _suf(U.dtype))(_p(U), u32(nf), _p(R), u32(nreg), u32(R.shape[1]), _p(P), _p(A), PT[ptype])
    return P, A


def poolrgn_bprop(U, R, P, A, ptype):
    R = _c(R, np.uint32); P = _c(P)
    nf = U.shape[1]
    getattr(lib(), "orc_poolrgn_bprop_" + _suf(U.dtype))(_p(U), u32(nf), _p(R), u32(R.shape[0]), u32(R.shape[1]), _p(P), _p(A), PT[ptype])
    return U


def scanpool(W, bias, relu, X, R, ptype, want_argmax=False):
    """corr1ord -> (+bias) -> (rectify) -> poolrgn in one pass."""
    W = _c(W); X = _c(X, np.uint8).ravel(); R = _c(R, np.uint32)
    bias = None if bias is None else _c(bias, W.dtype).ravel()
    m, nf = W.shape[0] // 4, W.shape[1]
    nreg = R.shape[0]
    P = np.empty((nreg, nf * (2 if ptype == "all" else 1)), W.dtype)
    A = np.empty((nreg, nf), np.uint32) if (want_argmax and ptype in ("max", "all")) else None
    getattr(lib(), "orc_scanpool_" + _suf(W.dtype))(
        _p(W), u32(m), u32(nf), _p(bias), int(bool(relu)), _p(X), u32(X.size),
        _p(R), u32(nreg), u32(R.shape[1]), _p(P), _p(A), PT[ptype])
    return P, A


# ------------------------------------------------------- elementwise pieces
def dropoutord_fp_tr(X, U, rate):
    X = _c(X, np.uint8).ravel(); U = _c(U, np.float32).ravel()
    Z = np.empty_like(X); M = np.empty(X.shape, np.uint8)
    lib().orc_dropoutord_fp_tr(_p(X), _p(U), ctypes.c_float(rate), _p(Z), _p(M), u32(X.size))
    return Z, M.astype(bool)


def gradstep(P, dP, drate, mP, mrate):
    getattr(lib(), "orc_gradstep_" + _suf(P.dtype))(_p(P), _p(dP), _p(drate), _p(mP), _p(mrate), u32(P.size))


def gradstep_nesterov1(P, mP, mrate):
    getattr(lib(), "orc_gradstep_nesterov1_" + _suf(P.dtype))(_p(P), _p(mP), _p(mrate), u32(P.size))


def gradstep_nesterov2(P, dP, drate, mP, mrate):
    getattr(lib(), "orc_gradstep_nesterov2_" + _suf(P.dtype))(_p(P), _p(dP), _p(drate), _p(mP), _p(mrate), u32(P.size))


def madd_bcast(A, b, k, dst):
    A = _c(A); b = _c(b, A.dtype).ravel()
    getattr(lib(), "orc_madd_bcast_" + _suf(A.dtype))(_p(A), _p(b), _p(dst), u32(A.size), u32(b.size), u32(k))


def maskout(M, A):
    M8 = _c(M, np.uint8)
    getattr(lib(), "orc_maskout_" + _suf(A.dtype))(_p(M8), _p(A), u32(A.size))


def calc_zmask(Z, M8):
    """M8 is a uint8 array the caller zeroed (loss.py:113); only 1s are written."""
    Z = _c(Z)
    getattr(lib(), "orc_calc_zmask_" + _suf(Z.dtype))(_p(Z), _p(M8), u32(Z.shape[0]), u32(Z.shape[1]))


def dropout_fp_tr(X, rate, U, matchrows=False):
    X = _c(X); rate = _c(rate, X.dtype).ravel(); U = _c(U, np.float32).ravel()
    Z = np.empty_like(X); M = np.empty(X.shape, np.uint8)
    m = rate.size; k = X.shape[1] // m
    if matchrows:
        getattr(lib(), "orc_dropout_fp_tr_match_" + _suf(X.dtype))(_p(X), _p(rate), _p(U), _p(Z), _p(M), u32(X.shape[0]), u32(X.shape[1]), u32(k))
    else:
        getattr(lib(), "orc_dropout_fp_tr_" + _suf(X.dtype))(_p(X), _p(rate), _p(U), _p(Z), _p(M), u32(X.size), u32(m), u32(k))
    return Z, M.astype(bool)


def dropout_fp_te(X, rate):
    X = _c(X); rate = _c(rate, X.dtype).ravel()
    Z = np.empty_like(X)
    getattr(lib(), "orc_dropout_fp_te_" + _suf(X.dtype))(_p(X), _p(rate), _p(Z), u32(X.size), u32(rate.size), u32(X.shape[1] // rate.size))
    return Z


def dropout_bp_tr(dZ, M):
    dZ = _c(dZ); M8 = _c(M, np.uint8)
    dX = np.empty_like(dZ)
    getattr(lib(), "orc_dropout_bp_tr_" + _suf(dZ.dtype))(_p(dZ), _p(M8), _p(dX), u32(dZ.size))
    return dX


def dropout_bp_te(dZ, rate):
    dZ = _c(dZ); rate = _c(rate, dZ.dtype).ravel()
    dX = np.empty_like(dZ)
    getattr(lib(), "orc_dropout_bp_te_" + _suf(dZ.dtype))(_p(dZ), _p(rate), _p(dX), u32(dZ.size), u32(rate.size), u32(dZ.shape[1] // rate.size))
    return dX


# ------------------------------------------------------- block-diagonal dots
def _bw(mode, nblock, xoff, xb, n, m, k, p, X, W, Z, beta_one=0):
    getattr(lib(), "orc_blockwise_" + _suf(W.dtype))(mode, nblock, xoff, int(xb), n, m, k, p, _p(X), _p(W), _p(Z), beta_one)


def blockwise_dot(X, W, nblock):
    """deepity_smat.blockwise_dot: Z[:,b] = X[:,b] . W[b]; X may be shared."""
    X = _c(X); W = _c(W)
    n = X.shape[0]; k = W.shape[0] // nblock; m = W.shape[1]
    Z = np.empty((n, m * nblock), X.dtype)
    _bw(0, nblock, 0, X.shape[1] * nblock == W.shape[0] and nblock > 1, n, m, k, k, X, W, Z)
    return Z


def blockwise_dot_nt(dZ, W, nblock):
    dZ = _c(dZ); W = _c(W)
    n = dZ.shape[0]; k = W.shape[0] // nblock; m = W.shape[1]
    dX = np.empty((n, W.shape[0]), dZ.dtype)
    _bw(1, nblock, 0, False, n, m, k, k, dX, W, dZ)
    return dX


def blockwise_dot_tn(X, dZ, nblock, W):
    X = _c(X); dZ = _c(dZ)
    n = X.shape[0]; k = W.shape[0] // nblock; m = W.shape[1]
    dW = np.empty_like(W)
    _bw(2, nblock, 0, X.shape[1] * nblock == W.shape[0] and nblock > 1, n, m, k, k, X, dW, dZ)
    return dW


def blockwise_dot_combined(Xs, W, nblock, Xbroadcast):
    """deepity_smat.py:206-216: sums the products of a list of inputs."""
    W = _c(W)
    n = Xs[0].shape[0]; m = W.shape[1]; p = W.shape[0] // nblock
    Z = np.empty((n, m * nblock), W.dtype)
    xoff = 0
    for X, xb in zip(Xs, Xbroadcast):
        if X is None:
            continue
        X = _c(X)
        k = X.shape[1] if xb else X.shape[1] // nblock
        _bw(0, nblock, xoff, xb, n, m, k, p, X, W, Z, beta_one=int(xoff != 0))
        xoff += k
    return Z


def blockwise_dot_nt_combined(Xs, dZ, W, nblock, Xbroadcast):
    W = _c(W); dZ = _c(dZ)
    n = dZ.shape[0]; m = W.shape[1]; p = W.shape[0] // nblock
    out = []; xoff = 0
    for X, xb in zip(Xs, Xbroadcast):
        if X is None:
            out.append(None); continue
        k = X.shape[1] if xb else X.shape[1] // nblock
        if not xb:
            dX = np.zeros_like(X)
            _bw(1, nblock, xoff, False, n, m, k, p, dX, W, dZ)
            out.append(dX)
        else:
            out.append(None)
        xoff += k
    return out


def blockwise_dot_tn_combined(Xs, dZ, W, nblock, Xbroadcast, dWmask=None):
    dZ = _c(dZ)
    n = dZ.shape[0]; m = W.shape[1]; p = W.shape[0] // nblock
    dW = np.zeros_like(W)
    xoff = 0
    for i, (X, xb) in enumerate(zip(Xs, Xbroadcast)):
        if X is None:
            continue
        X = _c(X)
        k = X.shape[1] if xb else X.shape[1] // nblock
        if dWmask is None or dWmask[i]:
            _bw(2, nblock, xoff, xb, n, m, k, p, X, dW, dZ)
        xoff += k
    return dW


# ------------------------------------------------- sequence batch assembly
_ORD = np.full(256, 255, np.uint8)
for _ch, _v in (("A", 0), ("C", 1), ("G", 2), ("T", 3), ("U", 3)):
    _ORD[ord(_ch)] = _v
    _ORD[ord(_ch.lower())] = _v
_COMP = {"A": "T", "C": "G", "G": "C", "T": "A", "U": "A", "N": "N",
         "a": "T", "c": "G", "g": "C", "t": "A", "u": "A", "n": "N"}


def acgt2ord(s):
    """kangaroo/util.py:50-56,68-74: ACGT/U -> 0123, everything else 255."""
    return _ORD[np.frombuffer(s.encode("latin-1"), np.uint8)]


def revcomp(s):
    """kangaroo/util.py:58-65,112-116: bytes outside ACGTUN become chr(255)."""
    return "".join(_COMP.get(ch, "\xff") for ch in s)[::-1]


def asbatch(seqs, padding, reverse_complement=False):
    """kangaroo/data.py:274-334: one minibatch -> (X uint8 [npos], R uint32 [n,2]).

    With reverse_complement the rows are interleaved fwd, rc, fwd, rc ...
    """
    if reverse_complement:
        seqs = [t for s in seqs for t in (s, revcomp(s))]
    cum = np.cumsum([0] + [padding + len(s) for s in seqs]).astype(np.uint32)
    R = np.stack([cum[:-1], cum[1:]], axis=1)
    X = acgt2ord(("." * padding).join([""] + list(seqs) + [""]))
    return X, R


def scan_windows(seq, windowsize, stride=1):
    """kangaroo/predict.py:281-284: the windows of one sequence in scan mode."""
    padseq = "N" * (windowsize - 1) + seq + "N" * (windowsize - 1)
    return [padseq[i:i + windowsize] for i in range(0, max(1, len(padseq) - windowsize + 1), stride)]


def predict(params, seqs, m, pool="max", nmodel=1, scan=None, stride=1, reverse_complement=False):
    """kangaroo/predict.py:168-196, 262-300, 434-452: direct scores, and in scan mode
    the per-sequence prediction maps with their max / mean / sum (NumPy reductions,
    as the reference takes them)."""
    X, R = asbatch(seqs, m - 1, reverse_complement)
    out = {"direct": score_net(params, X, R, pool, nmodel, strand_max=reverse_complement)}
    if scan:
        pmaps = []
        for s in seqs:
            Xw, Rw = asbatch(scan_windows(s, scan, stride), m - 1, reverse_complement)
            pmaps.append(score_net(params, Xw, Rw, pool, nmodel, strand_max=reverse_complement))
        out["pmaps"] = pmaps
        out["max"] = np.stack([p.max(axis=0) for p in pmaps])
        out["avg"] = np.stack([p.mean(axis=0) for p in pmaps])
        out["sum"] = np.stack([p.sum(axis=0) for p in pmaps])
    return out


# ------------------------------------------------------------- layer math
def logistic(x):
    """deepity/std/softmax.py:50-61 with one column per model; elemwise.py:112."""
    return 1.0 / (1.0 + np.exp(-x))


def bias_add(X, b):
    """deepity/std/elemwise.py:171: Z = X + b, b a row vector."""
    return (X + np.asarray(b, X.dtype).reshape(1, -1)).astype(X.dtype)


def relu(X):
    """deepity/std/elemwise.py:77: Z = maximum(0, X)."""
    return np.maximum(X, 0).astype(X.dtype)


def relu_bprop(dZ, Z):
    """deepity/std/elemwise.py:78: dX = dZ * sign(Z) with Z the rectified value."""
    return (dZ * np.sign(Z)).astype(dZ.dtype)


def loss(kind, Z, Y, Ymask=None, Zmask=None):
    """deepity/std/loss.py:52-65,98-112,125-147: (loss [ncol], dZ).  Elementwise term (Z-Y)^2
    (mse, scaled 1/2) or log(max(1e-15,Z))*Y + log(max(1e-15,1-Z))*(1-Y) (nll, negated), masked,
    mean over rows; dZ = (Z - Y), masked, times 1/nrow for both."""
    dt = Z.dtype
    if kind == "nll":
        L = np.log(np.maximum(1e-15, Z)) * Y + np.log(np.maximum(1e-15, 1 - Z)) * (1 - Y)
        scale = -1.0
    else:
        L = (Z - Y) ** 2
        scale = 0.5
    dZ = (Z - Y).astype(dt)
    for M in (Ymask, Zmask):
        if M is not None:
            L = np.where(M, L, 0)
            dZ = np.where(M, dZ, 0).astype(dt)
    return (scale * L.mean(axis=0)).astype(dt), (dZ * dt.type(1.0 / Z.shape[0])).astype(dt)


# -------------------------------------------------------- composite networks


def score_net(params, X, R, pool="max", nmodel=1, strand_max=False):
    """Forward scoring of ``nmodel`` independent DeepBind models.

    params: dict with Wscan [4m,16*I], bscan [16*I]; then either
      W1 [(P*I), 1], b1 [I]                                 (linear head), or
      W1 [(P*I), H], b1 [H*I], W2 [(H*I), 1], b2 [I]        (one hidden ReLU layer)
    where P = 16 (max/avg) or 32 (all) pooled features per model.
    Chain: deepity/std/full.py:78-83, elemwise.py:171,74-78; no output
    non-linearity (scores).  strand_max keeps max over row pairs
    (kangaroo/predict.py:145-164).  Returns [nseq, I].
    """
    I = nmodel
    pooled, _ = scanpool(params["Wscan"], params["bscan"], True, X, R, pool)
    h = blockwise_dot(pooled, params["W1"], I) + params["b1"].reshape(1, -1)
    if "W2" in params:
        h = np.maximum(h, 0)
        h = blockwise_dot(h, params["W2"], I) + params["b2"].reshape(1, -1)
    if strand_max:
        h = strand_max_rows(h, I)
    return h


def strand_max_rows(Z, I=1):
    """kangaroo/predict.py:144-164: rows are forward / reverse-complement pairs; the forward
    row is kept if it is >= the other, else the reverse-complement row."""
    Z = np.asarray(Z).reshape(-1, 2, I)
    return np.where(Z[:, 0] >= Z[:, 1], Z[:, 0], Z[:, 1])


def input_gradients(params, X, R, pool="max", nmodel=1, loss="mse", strand_max=False, dropout_rate=None):
    """Gradient maps of kangaroo.predict (predict.py:168-265 with deepity/node.py:317-338):
    the model output Z (after the logistic when the loss is nll) is fed back through a loss
    with target 0 and no minibatch mean, dZ = Z - 0 (loss.py:98-112), through the dense
    layers in test mode (full.py:84-89, dropout as scaling by 1 - rate), pooling
    (poolrgn_bprop), the rectifier and the scan (corr1ord.py:128-133) down to dX [npos, 4].
    With strand_max, of each forward / reverse-complement row pair only the row with the
    larger output feeds back (loss.py:113-117).  Returns (Z [nrow, I], dX)."""
    I = nmodel
    W, b = params["Wscan"], params["bscan"]
    act = np.maximum(corr1ord(W, X) + b.reshape(1, -1), 0)
    pooled, A = poolrgn(act, R, pool, True)
    pd = pooled if dropout_rate is None else dropout_fp_te(pooled, np.asarray(dropout_rate, pooled.dtype))
    h1 = blockwise_dot(pd, params["W1"], I) + params["b1"].reshape(1, -1)
    if "W2" in params:
        out = blockwise_dot(np.maximum(h1, 0), params["W2"], I) + params["b2"].reshape(1, -1)
    else:
        out = h1
    Z = 1.0 / (1.0 + np.exp(-out)) if loss == "nll" else out
    dZ = Z.copy()
    if strand_max:
        z = Z.reshape(-1, 2, I)
        keep = np.stack([z[:, 0] >= z[:, 1], ~(z[:, 0] >= z[:, 1])], 1).reshape(-1, I)
        dZ = np.where(keep, dZ, 0)
    if "W2" in params:
        dh = blockwise_dot_nt(dZ, params["W2"], I) * (h1 > 0)
    else:
        dh = dZ
    dpd = blockwise_dot_nt(dh, params["W1"], I)
    dpooled = dpd if dropout_rate is None else dropout_bp_te(dpd, np.asarray(dropout_rate, dpd.dtype))
    dact = poolrgn_bprop(np.zeros_like(act), R, np.ascontiguousarray(dpooled.astype(act.dtype)), A, pool) * (act > 0)
    dX = corr1ord_bprop_X(np.zeros((X.size, 4), W.dtype), W, np.ascontiguousarray(dact.astype(W.dtype)))
    return Z, dX


def train_grads(params, X, R, Y, pool="all", nmodel=1, loss="nll", dropmask=None,
                decay=None, Ymask=None, strand_pairs=False):
    """One forward/backward pass of the training graph; returns (loss[I], grads).

    Network: scan -> bias -> rectify -> pool -> dropout(mask given) ->
    full(H) -> bias -> rectify -> full(1) -> bias -> [logistic for nll] -> loss,
    or with no hidden layer when W2 is absent.  Backward follows
    deepity/std/loss.py:98-112 (dZ = (Z-Y)/nrow for both losses),
    full.py:84-89, elemwise.py:78,172-181, kangaroo/_ext/poolrgn.py:176-180,
    corr1ord.py:120-126.  decay: optional dict name -> per-model L1 weights
    (full.py:111-119, corr1ord.py:125-126).  strand_pairs: rows are forward /
    reverse-complement pairs; only the row with the larger output of each pair
    contributes to loss and gradient (loss.py:52-65,98-117 with maskout.cu:54-67),
    while the mean still divides by all rows.
    """
    I = nmodel
    dt = params["Wscan"].dtype
    m = params["Wscan"].shape[0] // 4
    nf = params["Wscan"].shape[1]
    X = _c(X, np.uint8).ravel()
    Z0 = corr1ord(params["Wscan"], X)
    A0 = relu(bias_add(Z0, params["bscan"]))
    pooled, amax = poolrgn(A0, R, pool, want_argmax=True)
    pd = pooled if dropmask is None else (pooled * dropmask).astype(dt)
    h1 = bias_add(blockwise_dot(pd, params["W1"], I).astype(dt), params["b1"])
    if "W2" in params:
        a1 = relu(h1)
        out = bias_add(blockwise_dot(a1, params["W2"], I).astype(dt), params["b2"])
    else:
        out = h1
    Yb = np.tile(_c(Y, dt).reshape(len(Y), -1), (1, I)) if Y.shape[-1] != I or Y.ndim == 1 else _c(Y, dt)
    nrow = out.shape[0]
    Zo = logistic(out).astype(dt) if loss == "nll" else out
    Zmask = None
    if strand_pairs:
        Zmask = np.zeros(Zo.shape, np.uint8)
        calc_zmask(Zo, Zmask)
        Zmask = Zmask.astype(bool)
    lossval, dout = globals()["loss"](loss, Zo, Yb, Ymask, Zmask)
    g = {}
    if "W2" in params:
        g["b2"] = dout.sum(axis=0).astype(dt)
        g["W2"] = blockwise_dot_tn(a1, dout, I, params["W2"])
        da1 = blockwise_dot_nt(dout, params["W2"], I)
        dh1 = relu_bprop(da1.astype(dt), a1)
    else:
        dh1 = dout
    g["b1"] = dh1.sum(axis=0).astype(dt)
    g["W1"] = blockwise_dot_tn(pd, dh1, I, params["W1"])
    dpd = blockwise_dot_nt(dh1, params["W1"], I)
    dpooled = dpd if dropmask is None else (dpd * dropmask).astype(dt)
    dA0 = np.zeros_like(A0)
    poolrgn_bprop(dA0, R, dpooled, amax, pool)
    dZ0 = relu_bprop(dA0, A0)
    g["bscan"] = dZ0.sum(axis=0).astype(dt)
    g["Wscan"] = corr1ord_bprop_W(np.zeros_like(params["Wscan"]), X, dZ0)
    if decay:
        for name, d in decay.items():
            W = params[name]
            d = _c(d, dt).ravel()
            # corr1ord.py:126 passes k = W.shape[0]/ninst, full.py:119 k = W.size/ninst
            k = W.shape[0] // I if name == "Wscan" else W.size // I
            madd_bcast(np.sign(W).astype(dt), d, k, g[name])
    return lossval.astype(dt), g


PARAM_ORDER = ("Wscan", "bscan", "W1", "b1", "W2", "b2")


def flatten(params):
    return np.concatenate([params[k].ravel() for k in PARAM_ORDER if k in params])


def unflatten(vec, like):
    out = {}; o = 0
    for k in PARAM_ORDER:
        if k in like:
            n = like[k].size
            out[k] = vec[o:o + n].reshape(like[k].shape)
            o += n
    return out


def nesterov_step(params, mom, drate, mrate, grad_fn):
    """deepity_smat.py:98-109 around gradstep.cu:52-72.  ``params``/``mom`` are
    flat vectors updated in place; grad_fn(P) returns the flat gradient."""
    gradstep_nesterov1(params, mom, mrate)
    dP = _c(grad_fn(params), params.dtype)
    gradstep_nesterov2(params, dP, drate, mom, mrate)
    return dP
