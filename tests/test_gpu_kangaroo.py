"""Parity of the kangaroo_smat entry points (called through the C ABI) with the
CPU oracle on seeded inputs.  Integer results and every float result whose
summation order the reference fixes are compared bit for bit; sums whose order
the reference leaves open (atomicAdd) are compared within 1e-5."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32


def rand_X(rng, n, n_frac=0.1, drop_frac=0.05):
    X = rng.integers(0, 4, size=n, dtype=np.uint8)
    u = rng.random(n)
    X[u < n_frac] = 255
    X[(u >= n_frac) & (u < n_frac + drop_frac)] = 254
    return X


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("m,nf,npos", [(1, 1, 7), (4, 3, 50), (5, 16, 333), (16, 17, 1000), (24, 16, 4099),
                                       (24, 48, 700), (24, 130, 513), (7, 64, 257)])
def test_corr1ord_bit_exact(cuda, orc, dtype, m, nf, npos):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(m * 1000 + nf)
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(dtype)
    X = rand_X(rng, npos)
    Z0 = rng.standard_normal((npos, nf)).astype(dtype)        # tail rows must survive
    want = orc.corr1ord(W, X, Z0.copy())
    Z = sm.asarray(Z0)
    ks.corr1ord(sm.asarray(W), sm.asarray(X), Z, 4)
    got = Z.asnumpy()
    assert np.array_equal(got, want)
    assert np.array_equal(got[npos - m + 1:], Z0[npos - m + 1:])


def test_corr1ord_input_shorter_than_filter_writes_nothing(cuda):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    W = np.ones((4 * 8, 2), f32)
    Z = sm.asarray(np.full((5, 2), 3.0, f32))
    ks.corr1ord(sm.asarray(W), sm.asarray(np.zeros(5, np.uint8)), Z, 4)
    assert np.all(Z.asnumpy() == 3.0)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("m,nf,npos", [(4, 3, 50), (24, 16, 4099), (16, 40, 900), (5, 1, 129)])
def test_corr1ord_bprop_W(cuda, orc, dtype, m, nf, npos):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(m + nf)
    X = rand_X(rng, npos)
    dZ = rng.standard_normal((npos, nf)).astype(dtype)
    dW0 = rng.standard_normal((4 * m, nf)).astype(dtype)       # accumulates into the caller's array
    want = orc.corr1ord_bprop_W(dW0.astype(np.float64), X, dZ.astype(np.float64))
    dW = sm.asarray(dW0)
    ks.corr1ord_bprop_W(dW, sm.asarray(X), sm.asarray(dZ), 4)
    got = dW.asnumpy()
    scale = np.abs(dZ).sum(axis=0).max()
    tol = 1e-5 if dtype == np.float32 else 1e-12
    assert np.max(np.abs(got - want)) <= tol * scale
    # deterministic: a second run gives the same bits
    dW2 = sm.asarray(dW0)
    ks.corr1ord_bprop_W(dW2, sm.asarray(X), sm.asarray(dZ), 4)
    assert np.array_equal(dW2.asnumpy(), got)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_corr1ord_bprop_X_bit_exact(cuda, orc, dtype):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(9)
    m, nf, n = 6, 5, 77
    W = rng.standard_normal((4 * m, nf)).astype(dtype)
    dZ = rng.standard_normal((n, nf)).astype(dtype)
    dX0 = rng.standard_normal((n, 4)).astype(dtype)
    want = orc.corr1ord_bprop_X(dX0.copy(), W, dZ)
    dX = sm.asarray(dX0)
    ks.corr1ord_bprop_X(dX, sm.asarray(W), sm.asarray(dZ), 4)
    assert np.array_equal(dX.asnumpy(), want)


def make_regions(rng, nreg, lo, hi, step=False):
    lens = rng.integers(lo, hi + 1, size=nreg)
    cum = np.concatenate([[0], np.cumsum(lens)])
    R = np.stack([cum[:-1], cum[1:]], axis=1).astype(np.uint32)
    if step:
        R = np.concatenate([R, rng.integers(1, 4, size=(nreg, 1)).astype(np.uint32)], axis=1)
    return R, int(cum[-1])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
@pytest.mark.parametrize("nf,step", [(16, False), (5, True), (130, False)])
def test_poolrgn_forward_and_backward(cuda, orc, dtype, ptype, nf, step):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(nf)
    R, nrow = make_regions(rng, 37, 1, 90, step)
    U = np.maximum(rng.standard_normal((nrow, nf)), 0).astype(dtype)   # many exact ties at 0
    P, A = orc.poolrgn(U, R, ptype, True)
    gP, gA = ks.poolrgn(sm.asarray(U), sm.asarray(R), ptype, want_argmax=ptype in ("max", "all"))
    assert np.array_equal(gP.asnumpy(), P)
    if A is not None:
        assert gA.dtype == np.uint32 and np.array_equal(gA.asnumpy(), A)
    else:
        assert gA is None
    dP = rng.standard_normal(P.shape).astype(dtype)
    want = orc.poolrgn_bprop(np.zeros_like(U), R, dP, A, ptype)
    dU = sm.zeros(U.shape, dtype)
    ks.poolrgn_bprop(dU, sm.asarray(R), sm.asarray(dP), gA, ptype)
    assert np.array_equal(dU.asnumpy(), want)


def test_poolrgn_bprop_overlapping_and_disjoint_regions(cuda, orc):
    """Disjoint ascending regions take plain read-modify-writes: two runs agree bit for bit and equal
    the oracle; overlapping (or descending) regions fall back to atomic adds and still give the sums."""
    import torch
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(5)
    nf, nrow = 16, 4000
    dis = np.array([[i * 40, i * 40 + 33] for i in range(100)], np.uint32)
    ovl = np.array([[0, 300], [100, 180], [150, 900], [2000, 2100], [1500, 2050]], np.uint32)
    for R, exact in ((dis, True), (ovl, False)):
        U0 = (rng.standard_normal((nrow, nf)) * 0.1).astype(f32)           # the operator accumulates into what is there
        act = np.maximum(rng.standard_normal((nrow, nf)), 0).astype(f32)
        P, A = orc.poolrgn(act, R, "all", True)
        dP = rng.standard_normal(P.shape).astype(f32)
        want = orc.poolrgn_bprop(U0.copy(), R, dP, A, "all")
        runs = []
        for _ in range(2):
            dU = sm.asarray(U0)
            ks.poolrgn_bprop(dU, sm.asarray(R), sm.asarray(dP), sm.asarray(A), "all")
            runs.append(dU.asnumpy())
        if exact:
            assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], want)
        else:
            assert np.max(np.abs(runs[0] - want)) <= 1e-5 * np.abs(want).max()


def test_poolrgn_validation_messages(cuda):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks, SmatException
    from deepbind_b200 import _lib
    from ctypes import byref
    U = sm.zeros((10, 4), f32); R = sm.asarray(np.array([[0, 10]], np.uint32))
    opt = _lib.c_poolrgn_options_t(); opt.ptype = 3
    bad = sm.zeros((1, 4), f32)
    with pytest.raises(SmatException, match='"all" pooling must have twice as many columns'):
        _lib.load().api_poolrgn(U._ptr, R._ptr, bad._ptr, None, byref(opt))
    opt.ptype = 1
    am = sm.zeros((1, 4), np.uint32)
    with pytest.raises(SmatException, match="pooledmaps_argmax can only be used for max/all pooling"):
        _lib.load().api_poolrgn(U._ptr, R._ptr, bad._ptr, am._ptr, byref(opt))
    opt.ptype = 0
    with pytest.raises(SmatException, match="pooledmaps_argmax must be specified for max pooling"):
        _lib.load().api_poolrgn_bprop(U._ptr, R._ptr, bad._ptr, None, byref(opt))
    R3 = sm.asarray(np.array([[0, 10, 1, 1]], np.uint32))
    with pytest.raises(SmatException, match="regions array must have 2 or 3 columns"):
        _lib.load().api_poolrgn(U._ptr, R3._ptr, bad._ptr, None, byref(opt))
    W = sm.zeros((8, 4), f32); X = sm.asarray(np.zeros(10, np.uint8)); Z = sm.zeros((10, 4), f32)
    with pytest.raises(SmatException, match="NotImplementedError: The given number of channels"):
        ks.corr1ord(W, X, Z, 2)
    Zbad = sm.zeros((9, 4), f32)
    with pytest.raises(SmatException, match="AssertionError"):
        ks.corr1ord(W, X, Zbad, 4)
    # the context is still usable after the errors
    ks.corr1ord(W, X, Z, 4)
    sm.sync()


def test_dropoutord(cuda, orc):
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(2)
    X = rand_X(rng, 5000, n_frac=0.2, drop_frac=0)
    U = rng.random(5000).astype(f32)
    Zw, Mw = orc.dropoutord_fp_tr(X, U, 0.3)
    Z, M = ks.dropoutord_fp_train(sm.asarray(X), 0.3, U=sm.asarray(U))
    assert np.array_equal(Z.asnumpy().ravel(), Zw) and np.array_equal(M.asnumpy().ravel(), Mw)
    # library-drawn mask: pads are always kept, about 30 % of the bases are dropped
    Z, M = ks.dropoutord_fp_train(sm.asarray(X), 0.3)
    z, mk = Z.asnumpy().ravel(), M.asnumpy().ravel()
    assert np.all(mk[X == 255]) and np.all(z[~mk] == 254) and np.array_equal(z[mk], X[mk])
    frac = 1 - mk[X != 255].mean()
    assert abs(frac - 0.3) < 0.03
