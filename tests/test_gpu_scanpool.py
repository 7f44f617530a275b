"""Parity of the fused scan+bias+rectify+pool kernels with the CPU oracle.

Forward: pooled values (max, mean, sum) and argmax indices are compared bit for
bit -- the kernel keeps the reference's tap order, row order and first-maximum
rule.  Backward: sums whose order the reference leaves to atomicAdd are compared
within 1e-5 of the magnitude of the summed terms."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32


def to_dev(*arrs):
    import torch
    out = []
    for a in arrs:
        if a is None:
            out.append(None)
        elif a.dtype == np.uint32:
            out.append(torch.from_numpy(a.view(np.int32)).cuda())
        else:
            out.append(torch.from_numpy(a).cuda())
    return out


def u32(t):
    return t.cpu().numpy().view(np.uint32)


CASES = [
    # m, nf, nseq, lmin, lmax, n_frac
    (24, 16, 64, 40, 40, 0.0),       # PBM-like
    (24, 16, 128, 101, 101, 0.0),    # ChIP-like minibatch
    (16, 16, 200, 20, 200, 0.05),    # ragged RNA with N
    (24, 48, 33, 1, 60, 0.1),        # sequences shorter than the filter
    (5, 7, 50, 1, 300, 0.2),         # generic filter length, nf not a multiple of 16
    (24, 130, 40, 30, 130, 0.0),     # several filter blocks, ragged tail block
    (11, 64, 9, 500, 900, 0.0),      # regions much longer than a tile
]


@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
@pytest.mark.parametrize("m,nf,nseq,lmin,lmax,n_frac", CASES)
def test_forward_bit_exact(cuda, orc, ptype, m, nf, nseq, lmin, lmax, n_frac):
    from deepbind_b200 import fused, synth
    X, R = synth.ragged_batch(nseq, lmin, lmax, m, seed=m * 7 + nf, n_frac=n_frac)
    rng = np.random.default_rng(nf)
    X[rng.random(X.size) < 0.02] = 254
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.0, nf).astype(f32)
    P, A = orc.scanpool(W, b, True, X, R, ptype, True)
    tW, tb, tX, tR = to_dev(W, b, X, R)
    gP, gA, gM = fused.scanpool(tW, tb, tX, tR, ptype, relu=True, want_argmax=True, want_actmask=True)
    assert np.array_equal(gP.cpu().numpy(), P)
    if A is not None:
        assert np.array_equal(u32(gA), A)
    # activity mask against the unfused chain
    Z = orc.corr1ord(W, X)
    act = np.maximum(Z + b, 0) > 0
    words = gM.cpu().numpy().view(np.uint16)
    bits = ((words[:, :, None] >> np.arange(16)) & 1).reshape(X.size, -1)[:, :nf].astype(bool)
    rows = np.zeros(X.size, bool)
    for r0, r1 in R:
        rows[r0:r1] = True
    assert np.array_equal(bits[rows], act[rows])


def test_forward_without_bias_or_rectifier(cuda, orc):
    from deepbind_b200 import fused, synth
    X, R = synth.ragged_batch(40, 5, 80, 8, seed=3)
    W = (np.random.default_rng(0).standard_normal((32, 20))).astype(f32)
    for bias, relu in ((None, False), (None, True)):
        P, A = orc.scanpool(W, bias, relu, X, R, "all", True)
        tW, tX, tR = to_dev(W, X, R)
        gP, gA, _ = fused.scanpool(tW, None, tX, tR, "all", relu=relu, want_argmax=True)
        assert np.array_equal(gP.cpu().numpy(), P) and np.array_equal(u32(gA), A)


def test_forward_regions_in_any_layout(cuda, orc):
    """Gaps, reversed order, overlaps and an empty region; rows past npos-m+1
    read as the zeros the unfused path leaves there."""
    from deepbind_b200 import fused
    rng = np.random.default_rng(8)
    m, nf, npos = 6, 16, 3000
    X = rng.integers(0, 4, size=npos, dtype=np.uint8)
    W = (rng.standard_normal((4 * m, nf)) * 0.2).astype(f32)
    b = rng.uniform(-0.2, 0.1, nf).astype(f32)
    R = np.array([[2900, 3000], [10, 50], [40, 45], [2000, 2001], [700, 1500], [60, 60], [0, 3], [2990, 2999],
                  [100, 101], [1500, 1501]], np.uint32)
    for ptype in ("max", "sum", "all"):
        P, A = orc.scanpool(W, b, True, X, R, ptype, True)
        tW, tb, tX, tR = to_dev(W, b, X, R)
        gP, gA, _ = fused.scanpool(tW, tb, tX, tR, ptype, want_argmax=True)
        assert np.array_equal(gP.cpu().numpy(), P, equal_nan=True)
        if A is not None:
            assert np.array_equal(u32(gA), A)


def test_all_zero_maps_pick_first_row(cuda):
    from deepbind_b200 import fused, synth
    X, R = synth.uniform_batch(10, 30, 24, seed=1)
    W = np.zeros((96, 16), f32); b = np.full(16, -1.0, f32)
    tW, tb, tX, tR = to_dev(W, b, X, R)
    gP, gA, _ = fused.scanpool(tW, tb, tX, tR, "max", want_argmax=True)
    assert np.all(gP.cpu().numpy() == 0)
    assert np.array_equal(u32(gA), R[:, :1] * 16 + np.arange(16, dtype=np.uint32))


@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
@pytest.mark.parametrize("m,nf,nseq,lmin,lmax,n_frac", CASES[:6])
def test_backward(cuda, orc, ptype, m, nf, nseq, lmin, lmax, n_frac):
    from deepbind_b200 import fused, synth
    X, R = synth.ragged_batch(nseq, lmin, lmax, m, seed=m + nf, n_frac=n_frac)
    rng = np.random.default_rng(nf + 1)
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.0, nf).astype(f32)
    # oracle chain in float64 on the float32 forward values
    Z = orc.corr1ord(W, X)
    act = np.maximum(Z + b, 0)
    P, A = orc.poolrgn(act, R, ptype, True)
    dP = rng.standard_normal(P.shape).astype(f32)
    dA = orc.poolrgn_bprop(np.zeros(act.shape, np.float64), R, dP.astype(np.float64), A, ptype)
    dZ = dA * np.sign(act)
    want_db = dZ.sum(axis=0)
    want_dW = orc.corr1ord_bprop_W(np.zeros((4 * m, nf)), X, dZ)
    tW, tb, tX, tR, tdP = to_dev(W, b, X, R, dP)
    gP, gA, gM = fused.scanpool(tW, tb, tX, tR, ptype, want_argmax=True, want_actmask=True)
    dW, db = fused.scanpool_bprop(m, nf, tX, tR, ptype, tdP, gA, gM)
    scale = np.abs(dZ).sum(axis=0).max() + 1e-30
    assert np.max(np.abs(dW.cpu().numpy() - want_dW)) <= 1e-5 * scale
    assert np.max(np.abs(db.cpu().numpy() - want_db)) <= 1e-5 * scale
    dW2, db2 = fused.scanpool_bprop(m, nf, tX, tR, ptype, tdP, gA, gM)
    assert np.array_equal(dW2.cpu().numpy(), dW.cpu().numpy()) and np.array_equal(db2.cpu().numpy(), db.cpu().numpy())


def test_fused_equals_unfused_device_chain(cuda):
    """The fused kernel and the drop-in operator chain agree bit for bit on the device."""
    import torch
    from deepbind_b200 import fused, synth, smat as sm, kangaroo_smat as ks, _lib
    X, R = synth.ragged_batch(300, 20, 200, 16, seed=12, n_frac=0.05)
    rng = np.random.default_rng(0)
    W = (rng.standard_normal((64, 16)) * 0.05).astype(f32); b = rng.uniform(-0.1, 0, 16).astype(f32)
    sW, sX, sR = sm.asarray(W), sm.asarray(X), sm.asarray(R)
    Z = sm.zeros((X.size, 16), f32)
    ks.corr1ord(sW, sX, Z, 4)
    tb = torch.from_numpy(b).cuda()
    dll = _lib.load()
    dll.db_bias_add(Z.data_ptr(), Z.data_ptr(), tb.data_ptr(), X.size, 16)
    dll.db_relu(Z.data_ptr(), Z.data_ptr(), Z.size)
    P, A = ks.poolrgn(Z, sR, "all", want_argmax=True)
    gP, gA, _ = fused.scanpool(sW.tensor, tb, sX.tensor.view(-1), sR.tensor, "all", want_argmax=True)
    assert torch.equal(gP, P.tensor) and torch.equal(gA, A.tensor)


def _backward_case(orc, m, nf, X, R, W, b, ptype):
    """Oracle chain (poolrgn_bprop -> rectifier -> filter gradient, float64 sums) beside the fused backward."""
    from deepbind_b200 import fused
    Z = orc.corr1ord(W, X)
    act = np.maximum(Z + b, 0)
    P, A = orc.poolrgn(act, R, ptype, True)
    rng = np.random.default_rng(5)
    dP = rng.standard_normal(P.shape).astype(f32)
    dA = orc.poolrgn_bprop(np.zeros(act.shape, np.float64), R, dP.astype(np.float64), A, ptype)
    dZ = dA * np.sign(act)
    want_db = dZ.sum(axis=0)
    want_dW = orc.corr1ord_bprop_W(np.zeros((4 * m, nf)), X, dZ)
    tW, tb, tX, tR, tdP = to_dev(W, b, X, R, dP)
    gP, gA, gM = fused.scanpool(tW, tb, tX, tR, ptype, want_argmax=True, want_actmask=True)
    assert np.array_equal(gP.cpu().numpy(), orc.scanpool(W, b, True, X, R, ptype, True)[0], equal_nan=True)
    dW, db = fused.scanpool_bprop(m, nf, tX, tR, ptype, tdP, gA, gM)
    scale = np.abs(dZ).sum(axis=0).max() + 1e-30
    assert np.max(np.abs(dW.cpu().numpy() - want_dW)) <= 1e-5 * scale
    assert np.max(np.abs(db.cpu().numpy() - want_db)) <= 1e-5 * scale


@pytest.mark.parametrize("ptype", ["max", "avg", "all"])
def test_backward_few_long_regions(cuda, orc, ptype):
    """Nine regions of 500-900 rows: several tiles per region group in the dense kernel, and
    the max-pooling kernel writing its results without a second stage."""
    from deepbind_b200 import synth
    m, nf = 11, 64
    X, R = synth.ragged_batch(9, 500, 900, m, seed=77)
    rng = np.random.default_rng(78)
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.0, nf).astype(f32)
    _backward_case(orc, m, nf, X, R, W, b, ptype)


def test_backward_max_regions_in_any_layout(cuda, orc):
    """Max pooling with gaps between regions, regions out of order, an empty region (its delta lands
    on the row the forward pass recorded for it, as in the reference) and rows past the last scan
    output (bias gradient only)."""
    rng = np.random.default_rng(9)
    m, nf, npos = 6, 40, 3000
    X = rng.integers(0, 4, size=npos, dtype=np.uint8)
    X[rng.random(npos) < 0.03] = 255
    W = (rng.standard_normal((4 * m, nf)) * 0.2).astype(f32)
    b = rng.uniform(-0.2, 0.1, nf).astype(f32)
    R = np.array([[2900, 3000], [10, 50], [2000, 2001], [700, 1500], [60, 60], [0, 3], [100, 101], [1500, 1501],
                  [1600, 1700], [1700, 1800], [1800, 1900], [200, 300], [300, 400], [400, 500], [500, 600], [600, 650],
                  [2100, 2200], [2200, 2300]], np.uint32)
    _backward_case(orc, m, nf, X, R, W, b, "max")


def test_full_size_ragged_both_strands(cuda, orc):
    """The ragged both-strand workload at its benchmark size (200,000 sequences of 20-200 nt with
    5 % N, 400,000 strands, 16 x 16 filters, strand max).  Swapping the two strands of every pair
    in the region list must not change a single score; sampled pairs are checked against the CPU
    oracle."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, nseq = 16, 200000
    p = synth.model_params(1, m, 51, "max")
    X, R = synth.ragged_batch(nseq, 20, 200, m, seed=52, n_frac=0.05, both_strands=True)
    net = DeepBindNet(p, 1, "max")
    tX, tR = to_dev(X, R)
    S = net.score(tX, tR, strand_max=True)
    assert S.shape == (nseq, 1)
    Rs = R.reshape(nseq, 2, 2)[:, ::-1].reshape(2 * nseq, 2).copy()
    S2 = net.score(tX, to_dev(Rs)[0], strand_max=True)
    assert torch.equal(S, S2)
    pick = np.random.default_rng(4).choice(nseq, 64, replace=False)
    rows = np.stack([2 * pick, 2 * pick + 1], 1).ravel()
    Xs = np.concatenate([X[R[i, 0]:R[i, 1]] for i in rows] + [np.full(m - 1, 255, np.uint8)])
    ends = np.cumsum([R[i, 1] - R[i, 0] for i in rows]).astype(np.uint32)
    Rp = np.stack([np.concatenate([[0], ends[:-1]]).astype(np.uint32), ends], 1)
    want = orc.score_net(p, Xs, Rp, "max", 1, strand_max=True)
    got = S[torch.from_numpy(pick).cuda()].cpu().numpy()
    assert np.max(np.abs(got - want)) <= 1e-6 * np.abs(want).max()
