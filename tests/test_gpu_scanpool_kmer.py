"""The k-mer scoring kernel (db_scanpool_score) against the exact FP32 kernel and the oracle.
It sums the taps in groups of two or three from k-mer tables, so its pooled values differ
from the tap-by-tap kernel by FP32 rounding of the regrouped sums only: the bound stated
here is 1e-6 of the largest activation (times the row count for sums)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32
TOL = 1e-6


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)).cuda()


@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
@pytest.mark.parametrize("m,nf,nseq,lmin,lmax", [(24, 16, 300, 101, 101), (16, 16, 500, 20, 200), (24, 48, 120, 30, 90),
                                                 (8, 7, 200, 3, 70), (12, 16, 150, 10, 40), (20, 33, 90, 25, 300),
                                                 (32, 16, 60, 40, 1000)])
def test_scoring_kernel_matches_exact_kernel_and_oracle(cuda, orc, ptype, m, nf, nseq, lmin, lmax):
    import torch
    from deepbind_b200 import fused, synth
    X, R = synth.ragged_batch(nseq, lmin, lmax, m, seed=m + nf, n_frac=0.05)
    rng = np.random.default_rng(nf)
    X[rng.random(X.size) < 0.02] = 254
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(f32)
    b = rng.uniform(-0.1, 0.05, nf).astype(f32)
    for relu in (True, False):
        exact, _, _ = fused.scanpool(dev(W), dev(b), dev(X), dev(R), ptype, relu=relu)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = fused.scanpool_score(dev(W), dev(b), dev(X), dev(R), ptype, relu=relu, status=status)
        assert int(status.item()) == 0
        scale = float(np.abs(W).sum(axis=0).max() / 4 * 1.0 + np.abs(b).max())           # bound of any activation
        act_max = float(fused.scanpool(dev(W), dev(b), dev(X), dev(R), "max", relu=False)[0].abs().max())
        bound = TOL * max(act_max, 1e-3) * (float((R[:, 1] - R[:, 0]).max()) if ptype == "sum" else 1.0)
        assert float((got - exact).abs().max()) <= bound, (relu, float((got - exact).abs().max()), bound)
    want, _ = orc.scanpool(W.astype(np.float64), b.astype(np.float64), True, X, R, ptype)
    got = fused.scanpool_score(dev(W), dev(b), dev(X), dev(R), ptype, relu=True).cpu().numpy()
    rows = float((R[:, 1] - R[:, 0]).max()) if ptype == "sum" else 1.0
    assert np.max(np.abs(got - want)) <= 1e-5 * max(np.abs(want).max(), 1e-3) + 1e-6 * rows


def test_region_shapes_the_tiles_do_not_like(cuda, orc):
    """Regions of one to three rows (more than 32 per 128-row tile), an empty region, gaps between
    regions, a region over twenty tiles, a region ending past the scanned rows."""
    import torch
    from deepbind_b200 import fused
    rng = np.random.default_rng(3)
    m, nf, npos = 8, 16, 6000
    X = rng.integers(0, 4, size=npos, dtype=np.uint8)
    X[rng.random(npos) < 0.05] = 255
    W = (rng.standard_normal((4 * m, nf)) * 0.2).astype(f32)
    b = rng.uniform(-0.2, 0.1, nf).astype(f32)
    R = []
    pos = 0
    for i in range(150):                                   # 150 tiny regions back to back
        n = int(rng.integers(1, 4)); R.append((pos, pos + n)); pos += n
    R.append((pos + 5, pos + 5))                           # empty: reads its first row, count 0
    R.append((pos + 40, pos + 40 + 2700))                  # twenty-one tiles
    pos = pos + 40 + 2700 + 300                            # a gap of 300 unscored rows
    R.append((pos, pos + 17))
    R.append((5950, 5999))                                 # rows past npos - m + 1 read as zero activations
    R = np.asarray(R, np.uint32)
    for ptype in ("max", "all", "sum"):
        exact, _, _ = fused.scanpool(dev(W), dev(b), dev(X), dev(R), ptype)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = fused.scanpool_score(dev(W), dev(b), dev(X), dev(R), ptype, status=status)
        assert int(status.item()) == 0
        e, g = exact.cpu().numpy(), got.cpu().numpy()
        ok = np.isfinite(e)
        assert np.array_equal(np.isfinite(g), ok)          # the empty region's mean is x/0 in both
        assert np.max(np.abs(g[ok] - e[ok])) <= 1e-6 * max(1.0, np.abs(e[ok]).max()) * (2700 if ptype == "sum" else 1)


def test_overlapping_regions_are_reported(cuda):
    import torch
    from deepbind_b200 import fused
    X = np.zeros(3000, np.uint8)
    W = np.zeros((96, 16), f32)
    for R in ([[0, 200], [100, 300]], [[500, 600], [0, 100]]):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        fused.scanpool_score(dev(W), None, dev(X), dev(np.asarray(R, np.uint32)), "max", status=status)
        assert int(status.item()) == 3
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fused.scanpool_score(dev(W), None, dev(X), dev(np.asarray([[0, 100], [100, 100], [100, 250]], np.uint32)), "max", status=status)
    assert int(status.item()) == 0


def test_net_score_uses_the_scoring_kernel_and_stays_partition_independent(cuda, orc):
    """DeepBindNet.score: k-mer path by default, exact on request; scoring a batch in chunks gives
    the same bits as scoring it whole (a region's sum runs over its rows in order whatever the tiles)."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, I = 16, 3
    p = synth.model_params(I, m, 4, "all")
    net = DeepBindNet(p, I, "all")
    Xh, Rh = synth.ragged_batch(5000, 20, 200, m, seed=8, n_frac=0.05, both_strands=True)
    X, R = dev(Xh), dev(Rh)
    fast, exact = net.score(X, R, strand_max=True), net.score(X, R, strand_max=True, exact=True)
    assert fast.shape == (5000, I)
    assert float((fast - exact).abs().max()) <= 2e-6 * float(exact.abs().max())
    want = orc.score_net({k: v.astype(np.float64) for k, v in p.items()}, Xh, Rh, "all", I, strand_max=True)
    assert np.max(np.abs(fast.cpu().numpy() - want)) <= 1e-5 * np.abs(want).max()
    whole = net.score(X, R)
    parts = torch.cat([net.score(X, R[lo:lo + 1234]) for lo in range(0, R.shape[0], 1234)])
    assert torch.equal(whole, parts)
