"""Parity of the tensor-core (tcgen05) many-model scan with the CPU oracle.

The one-hot operand is exact in bf16 and f16; the weights carry 8, 16 or 24
significant bits as 1, 2, 3 bf16 pieces (precision 1, 2, 3), or 22 / 11 bits as
2 / 1 f16 pieces of prescaled weights (precision 4, 5).  A weight's rounding
error is the same at every position, so it does not average out under mean
pooling: the tolerance is stated relative to the largest activation of the layer
(the largest max-pooled value), times the number of rows for sum pooling: 2e-3
for one bf16 piece (the bound set for bf16/TF32 paths), 5e-4 for one f16 piece,
1e-5 for bf16x2, bf16x3 (the fp32 bound) and 3e-6 for f16x2."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32
TOL = {1: 2e-3, 2: 1e-5, 3: 1e-5, 4: 3e-6, 5: 5e-4}


def dev(a):
    import torch
    if a is None:
        return None
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).cuda()


CASES = [
    # m, nmodel, nseq, lmin, lmax, n_frac
    (24, 8, 64, 101, 101, 0.0),      # one filter tile, ChIP-like
    (24, 20, 50, 40, 40, 0.0),       # three tiles, the last one half empty
    (16, 8, 80, 20, 200, 0.05),      # ragged RNA with N: tiles of 36..215 positions
    (24, 9, 30, 200, 400, 0.0),      # regions spanning several 128-column tiles
    (10, 8, 40, 5, 60, 0.1),         # filter length not a multiple of 4 (zero-padded taps)
    (16, 1, 300, 20, 200, 0.05),     # one model: the 16 filters repeated in every lane quarter, regions shared by all warps
    (24, 2, 200, 101, 101, 0.0),     # two models (32 filters), equal lengths: still flat tiles
]


@pytest.mark.parametrize("nsplit", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
@pytest.mark.parametrize("m,nmodel,nseq,lmin,lmax,n_frac", CASES)
def test_pooled_matches_oracle(cuda, orc, nsplit, ptype, m, nmodel, nseq, lmin, lmax, n_frac):
    from deepbind_b200 import fused, synth
    nf = 16 * nmodel
    X, R = synth.ragged_batch(nseq, lmin, lmax, m, seed=m + nmodel, n_frac=n_frac)
    rng = np.random.default_rng(nmodel)
    X[rng.random(X.size) < 0.01] = 254
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.0, nf).astype(f32)
    want, _ = orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, ptype)
    tcw = fused.TCWeights(dev(W), dev(b), nsplit)
    got, _ = fused.scanpool_tc(tcw, dev(X), dev(R), ptype)
    got = got.cpu().numpy()
    assert got.shape == want.shape
    scale = np.abs(orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, "max")[0]).max()
    if ptype == "sum":
        scale *= (R[:, 1] - R[:, 0]).max()
    assert np.max(np.abs(got - want)) <= TOL[nsplit] * scale, (np.max(np.abs(got - want)), scale)


@pytest.mark.parametrize("nsplit", [1, 3, 4, 5])
@pytest.mark.parametrize("ptype", ["max", "all"])
def test_fused_linear_head_scores(cuda, orc, nsplit, ptype):
    from deepbind_b200 import fused, synth
    m, I = 24, 24
    X, R = synth.uniform_batch(300, 101, m, seed=3)
    p = synth.model_params(I, m, 4, ptype)
    p64 = {k: v.astype(np.float64) for k, v in p.items()}
    want = orc.score_net(p64, X, R, ptype, I)
    tcw = fused.TCWeights(dev(p["Wscan"]), dev(p["bscan"]), nsplit)
    pooled, scores = fused.scanpool_tc(tcw, dev(X), dev(R), ptype, headW=dev(p["W1"].ravel()), headB=dev(p["b1"]),
                                       want_pooled=True)
    scale = np.abs(want).max()
    assert np.max(np.abs(scores.cpu().numpy() - want)) <= TOL[nsplit] * scale
    wp, _ = orc.scanpool(p64["Wscan"], p64["bscan"], True, X, R, ptype)
    assert np.max(np.abs(pooled.cpu().numpy() - wp)) <= TOL[nsplit] * np.abs(wp).max()


def test_three_pieces_agree_with_fp32_kernel(cuda):
    """bf16x3 against the bit-exact FP32 lookup-add kernel on the device."""
    import torch
    from deepbind_b200 import fused, synth
    m, I = 24, 40
    X, R = synth.uniform_batch(2000, 101, m, seed=9)
    p = synth.model_params(I, m, 10, "all")
    W, b, dX, dR = dev(p["Wscan"]), dev(p["bscan"]), dev(X), dev(R)
    ref, _, _ = fused.scanpool(W, b, dX, dR, "all")
    got, _ = fused.scanpool_tc(fused.TCWeights(W, b, 3), dX, dR, "all")
    assert float((got - ref).abs().max()) <= 1e-5 * float(ref.abs().max())


@pytest.mark.parametrize("wscale", [1e-6, 0.05, 300.0])
def test_f16_prescale_covers_small_and_large_weights(cuda, orc, wscale):
    """f16 pieces hold weights of any magnitude: the bank is prescaled by a power of two."""
    from deepbind_b200 import fused, synth
    m, nf = 24, 128
    X, R = synth.ragged_batch(60, 30, 120, m, seed=5, n_frac=0.03)
    rng = np.random.default_rng(6)
    W = (rng.standard_normal((4 * m, nf)) * wscale).astype(f32)
    b = (rng.uniform(-2.0, 0.0, nf) * wscale).astype(f32)
    want, _ = orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, "all")
    scale = np.abs(want[:, 0::2]).max()
    for precision, tol in (("f16x2", 3e-6), ("f16", 5e-4)):
        got, _ = fused.scanpool_tc(fused.TCWeights(dev(W), dev(b), precision), dev(X), dev(R), "all")
        assert np.max(np.abs(got.cpu().numpy() - want)) <= tol * scale, precision


@pytest.mark.parametrize("ptype", ["max", "all"])
@pytest.mark.parametrize("m,L,nseq,gap", [(24, 101, 3000, 0),     # 124-row regions, two per tile: the benchmark's shape
                                          (24, 40, 2500, 0),      # four 63-row regions per tile
                                          (16, 20, 900, 0),       # seven 35-row regions per tile: a warp owns two regions of one tile
                                          (24, 233, 700, 0),      # 256 rows: one region fills a tile
                                          (24, 150, 900, 0),      # one region per tile, tiles 173 rows apart
                                          (24, 234, 300, 0),      # 257 rows: too long for a tile, flat tiles take over
                                          (8, 30, 1500, 5),       # equal regions with equal gaps between them
                                          (24, 101, 5, 0), (24, 101, 1, 0)])
def test_equal_length_batches_take_region_aligned_tiles(cuda, orc, ptype, m, L, nseq, gap):
    """Equal-length batches run the kernel's region-aligned tiling (whole regions per
    accumulator tile); the answers must be those of the oracle all the same, across many
    tiles, operand stages and CTAs."""
    from deepbind_b200 import fused
    I = 8
    nf = 16 * I
    rng = np.random.default_rng(m * L + nseq)
    P = L + m - 1
    S = P + gap
    X = np.full(nseq * S + m - 1 + gap, 255, np.uint8)
    R = np.empty((nseq, 2), np.uint32)
    for i in range(nseq):
        R[i] = (i * S, i * S + P)
        X[i * S + m - 1:i * S + P] = rng.integers(0, 4, L)
    X[rng.random(X.size) < 0.01] = 254
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.05, nf).astype(f32)
    want, _ = orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, ptype)
    hW = rng.standard_normal(I * (32 if ptype == "all" else 16)).astype(f32); hB = rng.standard_normal(I).astype(f32)
    for prec in (4, 1):
        tcw = fused.TCWeights(dev(W), dev(b), prec)
        got, scores = fused.scanpool_tc(tcw, dev(X), dev(R), ptype, headW=dev(hW), headB=dev(hB), want_pooled=True)
        scale = np.abs(want).max()
        assert np.max(np.abs(got.cpu().numpy() - want)) <= TOL[prec] * scale, prec
        ws = (want.reshape(nseq, I, -1) * hW.reshape(I, -1)).sum(axis=2) + hB
        assert np.max(np.abs(scores.cpu().numpy() - ws)) <= TOL[prec] * scale * np.abs(hW.reshape(I, -1)).sum(axis=1).max(), prec


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable(cuda):
    """The kernel's waits are bounded.  With the operand encoders told never to announce
    their stage (a test switch of the library) and a deadline of a millisecond, the MMA
    issuer's first wait runs out with nothing in flight: the launch ends with status 1
    (raised as an exception here) and the next ordinary launch gives correct results."""
    import torch
    from deepbind_b200 import _lib, fused, synth, SmatException
    dll = _lib.load()
    m, I = 24, 8
    X, R = synth.uniform_batch(400, 101, m, seed=2)
    p = synth.model_params(I, m, 3, "all")
    tcw = fused.TCWeights(dev(p["Wscan"]), dev(p["bscan"]), "f16x2")
    good, _ = fused.scanpool_tc(tcw, dev(X), dev(R), "all")
    dll.db_scanpool_tc_debug(2_000_000, 1)
    try:
        with pytest.raises(SmatException, match="timed out"):
            fused.scanpool_tc(tcw, dev(X), dev(R), "all")
    finally:
        dll.db_scanpool_tc_debug(0, 0)
    torch.cuda.synchronize()
    again, _ = fused.scanpool_tc(tcw, dev(X), dev(R), "all")
    assert torch.equal(again, good)
    Xr, Rr = synth.ragged_batch(300, 20, 150, m, seed=4)          # and the flat-tile path
    dll.db_scanpool_tc_debug(2_000_000, 1)
    try:
        with pytest.raises(SmatException, match="timed out"):
            fused.scanpool_tc(tcw, dev(Xr), dev(Rr), "all")
    finally:
        dll.db_scanpool_tc_debug(0, 0)
    ok, _ = fused.scanpool_tc(tcw, dev(Xr), dev(Rr), "all")
    assert bool(torch.isfinite(ok).all())


@pytest.mark.parametrize("bad", [np.inf, -np.inf, np.nan])
def test_a_filter_bank_with_a_non_finite_weight_is_refused(cuda, bad):
    """max |W| sets the f16 prescale and the bound of the saturating rectifier, so an Inf or
    NaN weight cannot be scanned: preparing the bank records it, the scan writes nothing and
    reports status 4."""
    import torch
    from deepbind_b200 import fused, synth, SmatException
    m, I = 24, 8
    X, R = synth.uniform_batch(64, 101, m, seed=2)
    p = synth.model_params(I, m, 3, "all")
    W = p["Wscan"].copy()
    W[17, 5] = bad
    tcw = fused.TCWeights(dev(W), dev(p["bscan"]), "f16x2")
    with pytest.raises(SmatException, match="Inf or NaN"):
        fused.scanpool_tc(tcw, dev(X), dev(R), "all")
    good = fused.TCWeights(dev(p["Wscan"]), dev(p["bscan"]), "f16x2")
    out, _ = fused.scanpool_tc(good, dev(X), dev(R), "all")
    assert bool(torch.isfinite(out).all())


def test_gaps_between_regions_and_tail_rows(cuda, orc):
    from deepbind_b200 import fused
    rng = np.random.default_rng(8)
    m, nf, npos = 8, 128, 3000
    X = rng.integers(0, 4, size=npos, dtype=np.uint8)
    W = (rng.standard_normal((4 * m, nf)) * 0.2).astype(f32)
    b = rng.uniform(-0.2, 0.1, nf).astype(f32)
    # ascending, with gaps; the last regions reach rows past npos-m+1, which read as zero
    R = np.array([[0, 3], [10, 50], [50, 51], [700, 1500], [1500, 1501], [2000, 2001], [2900, 2990], [2990, 2999]], np.uint32)
    want, _ = orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, "all")
    got, _ = fused.scanpool_tc(fused.TCWeights(dev(W), dev(b), 3), dev(X), dev(R), "all")
    assert np.max(np.abs(got.cpu().numpy() - want)) <= 1e-5 * np.abs(want).max()


def test_regions_out_of_order_are_reported(cuda):
    from deepbind_b200 import fused, SmatException
    X = np.zeros(5000, np.uint8); R = np.array([[100, 200], [0, 100]], np.uint32)
    W = np.zeros((96, 16), f32)
    with pytest.raises(SmatException, match="ascend without overlap"):
        fused.scanpool_tc(fused.TCWeights(dev(W), None, 1), dev(X), dev(R), "max")
    # the device is still usable
    got, _ = fused.scanpool_tc(fused.TCWeights(dev(W), None, 1), dev(X), dev(np.array([[0, 100]], np.uint32)), "max")
    assert float(got.abs().max()) == 0.0


def test_many_sequences_many_ctas(cuda, orc):
    """Enough sequences for several stages per CTA and several CTAs per filter tile."""
    from deepbind_b200 import fused, synth
    m, I = 24, 16
    X, R = synth.ragged_batch(6000, 30, 150, m, seed=77, n_frac=0.02)
    p = synth.model_params(I, m, 78, "all")
    want, _ = orc.scanpool(p["Wscan"].astype(np.float64), p["bscan"].astype(np.float64), True, X, R, "all")
    got, _ = fused.scanpool_tc(fused.TCWeights(dev(p["Wscan"]), dev(p["bscan"]), 3), dev(X), dev(R), "all")
    assert np.max(np.abs(got.cpu().numpy() - want)) <= 1e-5 * np.abs(want).max()


def test_full_size_genome_scan(cuda, orc):
    """The benchmark's own size: 1,000,000 sequences x 101 nt scored by 512 models in one launch
    (score matrix 2 GB).  The second half of the batch repeats the first, so the two halves of the
    score matrix must agree (to the mean pooling's grouping: a sequence's rows fall differently on
    the kernel's column pieces); sampled rows are checked against the CPU oracle; per-model column
    sums of the two halves give a checksum over every score."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, I, L, half = 24, 512, 101, 500000
    p = synth.model_params(I, m, 7, "all")
    Xh, Rh = synth.uniform_batch(half, L, m, seed=11)
    rows = half * (L + m - 1)
    X2 = np.concatenate([Xh[:rows], Xh[:rows], np.full(m - 1, 255, np.uint8)])
    R2 = np.concatenate([Rh, Rh + np.uint32(rows)]).astype(np.uint32)
    net = DeepBindNet(p, I, "all")
    net.prepare_tc("f16x2")
    X, R = dev(X2), dev(R2)
    S = net.score_tc(X, R)
    assert S.shape == (2 * half, I) and bool(torch.isfinite(S).all())
    scale = float(S.abs().max())
    assert float((S[:half] - S[half:]).abs().max()) <= 2e-6 * scale
    ca, cb = S[:half].double().sum(0), S[half:].double().sum(0)
    assert float((ca - cb).abs().max()) <= 1e-7 * float(S[:half].double().abs().sum(0).max())
    pick = np.random.default_rng(3).choice(half, 24, replace=False)
    Xs = np.concatenate([Xh[Rh[i, 0]:Rh[i, 1]] for i in pick] + [np.full(m - 1, 255, np.uint8)])
    Rs = (np.arange(24, dtype=np.uint32)[:, None] * np.uint32(L + m - 1) + np.array([0, L + m - 1], np.uint32)).astype(np.uint32)
    want = orc.score_net({k: v.astype(np.float64) for k, v in p.items()}, Xs, Rs, "all", I)
    got = S[torch.from_numpy(pick).cuda()].cpu().numpy()
    assert np.max(np.abs(got - want)) <= 3e-6 * max(scale, np.abs(want).max())
    assert np.max(np.abs(S[torch.from_numpy(pick + half).cuda()].cpu().numpy() - want)) <= 3e-6 * max(scale, np.abs(want).max())


def test_one_model_ragged_strand_max_against_the_exact_kernel(cuda):
    """The ragged both-strand scoring of a single 16-filter model through the tensor-core scan
    (fp32-grade pieces) against the bit-exact FP32 kernel: scores after the strand maximum."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    p = synth.model_params(1, 16, 51, "max")
    Xh, Rh = synth.ragged_batch(6000, 20, 200, 16, seed=52, n_frac=0.05, both_strands=True)
    net = DeepBindNet(p, 1, "max")
    X, R = dev(Xh), dev(Rh)
    exact = net.score(X, R, strand_max=True)
    for prec, tol in (("f16x2", 3e-6), ("bf16x3", 1e-5)):
        net.prepare_tc(prec)
        got = net.score_tc(X, R, strand_max=True)
        assert got.shape == exact.shape == (6000, 1)
        assert float((got - exact).abs().max()) <= tol * float(exact.abs().max()), prec
