"""The scoring driver against the oracle's restatement of kangaroo.predict:
direct mode and scan mode (windowed prediction maps, their max / mean / sum),
one and several models, one and both strands."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ACGTN = np.frombuffer(b"ACGTN", dtype=np.uint8)


def seqs_of(rng, nseq, lmin, lmax):
    return [ACGTN[rng.choice(5, size=rng.integers(lmin, lmax + 1), p=[.24, .24, .24, .24, .04])].tobytes().decode() for _ in range(nseq)]


@pytest.mark.parametrize("rc", [False, True])
@pytest.mark.parametrize("I,pool,hidden", [(1, "max", 0), (3, "all", 0), (2, "all", 32)])
def test_direct_scores(cuda, orc, I, pool, hidden, rc):
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import predict
    rng = np.random.default_rng(3 + I)
    m = 24
    seqs = seqs_of(rng, 150, 20, 130)
    p = synth.model_params(I, m, 9, pool, hidden=hidden)
    want = orc.predict(p, seqs, m, pool, I, reverse_complement=rc)["direct"]
    got = predict(DeepBindNet(p, I, pool), seqs, reverse_complement=rc)
    assert sorted(got) == ["direct"]
    np.testing.assert_allclose(got["direct"].cpu().numpy(), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("rc", [False, True])
@pytest.mark.parametrize("I,W,stride", [(1, 20, 1), (4, 30, 5)])
def test_scan_mode(cuda, orc, I, W, stride, rc):
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import predict
    rng = np.random.default_rng(11 + W)
    m = 16
    seqs = seqs_of(rng, 40, 5, 260)
    p = synth.model_params(I, m, 12, "max")
    want = orc.predict(p, seqs, m, "max", I, scan=W, stride=stride, reverse_complement=rc)
    got = predict(DeepBindNet(p, I, "max"), seqs, scan=W, stride=stride, reverse_complement=rc, want_pmaps=True, max_windows=3000)
    np.testing.assert_allclose(got["direct"].cpu().numpy(), want["direct"], rtol=1e-5, atol=1e-6)
    assert len(got["pmaps"]) == len(seqs)
    for a, b in zip(got["pmaps"], want["pmaps"]):
        np.testing.assert_allclose(a.cpu().numpy(), b, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["max"].cpu().numpy(), want["max"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["sum"].cpu().numpy(), want["sum"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got["avg"].cpu().numpy(), want["avg"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("nseq", [500, 40000])
def test_predict_host_equals_device_scoring(cuda, nseq):
    """Host buffers in, host scores out: the small single-launch path and the
    pipelined path (scan pieces overlapped with the read-back) give what scoring
    the resident batch gives."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    I, m = 8, 24
    net = DeepBindNet(synth.model_params(I, m, 5, "all"), I, "all")
    Xh, Rh = synth.uniform_batch(nseq, 50, m, seed=2)
    X_host = torch.from_numpy(Xh).pin_memory(); R_host = torch.from_numpy(Rh.view(np.int32)).pin_memory()
    out_host = torch.empty((nseq, I), dtype=torch.float32).pin_memory()
    net.prepare_tc("f16x2")
    net.predict_host(X_host, R_host, out_host, tc=True)
    want = net.score_tc(X_host.cuda(), R_host.cuda()).cpu()
    # the mean-pooling sum of a region is grouped by where the 256-row tiles cut it, which depends on
    # the piece a sequence falls in: same values up to the order of FP32 additions
    assert float((out_host - want).abs().max()) <= 1e-6 * float(want.abs().max())
    exact = net.score(X_host.cuda(), R_host.cuda()).cpu()
    assert float((out_host - exact).abs().max()) <= 3e-6 * float(exact.abs().max()) * 4
    out2 = torch.empty_like(out_host)
    net.predict_host(X_host, R_host, out2, tc=False)
    assert torch.equal(out2, exact)
