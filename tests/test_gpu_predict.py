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


@pytest.mark.parametrize("precision,tol", [("f16x2", 3e-6), ("bf16x3", 1e-5), ("f16", 5e-4)])
@pytest.mark.parametrize("I,pool,hidden,rc", [(1, "max", 0, True), (3, "all", 0, False), (2, "all", 32, True)])
def test_tensor_core_precisions_of_the_driver(cuda, orc, precision, tol, I, pool, hidden, rc):
    """predict(precision=...) scores through the tensor-core scan: direct and scan mode against
    the oracle, tolerance relative to the largest score of the call."""
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import predict
    rng = np.random.default_rng(17 + I)
    m = 24
    seqs = seqs_of(rng, 120, 20, 130)
    p = synth.model_params(I, m, 9, pool, hidden=hidden)
    want = orc.predict(p, seqs, m, pool, I, scan=40, stride=7, reverse_complement=rc)
    got = predict(DeepBindNet(p, I, pool), seqs, scan=40, stride=7, reverse_complement=rc, precision=precision)
    for k in ("direct", "max", "avg"):
        w = np.asarray(want[k])
        assert np.abs(got[k].cpu().numpy() - w).max() <= 4 * tol * np.abs(w).max() + 1e-6, k


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


def test_predict_host_streamed_batches(cuda):
    """Three different batches streamed through the same device buffers with wait=False: each
    batch's host scores equal one device launch on that batch (the pieces of a call wait only for
    the same pieces of the call before), and a later call with other cuts first drains the pipe."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, I, nseq = 24, 16, 40000
    net = DeepBindNet(synth.model_params(I, m, 7, "all"), I, "all")
    net.prepare_tc("f16x2")
    dev_bufs = None
    hosts = []
    for seed in (1, 2, 3):
        Xh, Rh = synth.uniform_batch(nseq, 60, m, seed=seed)
        hosts.append((torch.from_numpy(Xh).pin_memory(), torch.from_numpy(Rh.view(np.int32)).pin_memory(),
                      torch.empty((nseq, I), dtype=torch.float32).pin_memory()))
    X = torch.empty(hosts[0][0].shape, dtype=torch.uint8, device=cuda)
    R = torch.empty(hosts[0][1].shape, dtype=torch.int32, device=cuda)
    out = torch.empty((nseq, I), dtype=torch.float32, device=cuda)
    for Xh, Rh, oh in hosts:
        net.predict_host(Xh, Rh, oh, dev_bufs=(X, R, out), tc=True, npiece=8, wait=False)
    net.predict_host_wait()
    for Xh, Rh, oh in hosts:
        want = net.score_tc(Xh.cuda(), Rh.cuda())
        assert torch.equal(oh, want.cpu())
    # other cuts on the same buffers: the pending calls are completed first
    net.predict_host(hosts[0][0], hosts[0][1], hosts[0][2], dev_bufs=(X, R, out), tc=True, npiece=8, wait=False)
    net.predict_host(hosts[1][0], hosts[1][1], hosts[1][2], dev_bufs=(X, R, out), tc=True, npiece=5)
    assert torch.equal(hosts[1][2], net.score_tc(hosts[1][0].cuda(), hosts[1][1].cuda()).cpu())
    assert torch.equal(hosts[0][2], net.score_tc(hosts[0][0].cuda(), hosts[0][1].cuda()).cpu())


@pytest.mark.parametrize("hidden,rate,I", [(32, 0.5, 3), (32, None, 2), (0, 0.25, 2)])
def test_predict_host_tensor_core_with_a_dense_head(cuda, hidden, rate, I):
    """Nets whose head is not the in-kernel linear one (hidden layer, test-mode dropout)
    take the pooled-features branch of the tensor-core path; the caller's buffers must
    still receive the scores."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, nseq = 24, 500
    net = DeepBindNet(synth.model_params(I, m, 7, "all", hidden=hidden), I, "all", loss="nll")
    if rate is not None:
        net.set_dropout(rate)
    Xh, Rh = synth.uniform_batch(nseq, 60, m, seed=4)
    X_host = torch.from_numpy(Xh).pin_memory(); R_host = torch.from_numpy(Rh.view(np.int32)).pin_memory()
    out_host = torch.full((nseq, I), float("nan"), dtype=torch.float32).pin_memory()
    net.prepare_tc("f16x2")
    net.predict_host(X_host, R_host, out_host, tc=True)
    exact = net.score(X_host.cuda(), R_host.cuda()).cpu()
    assert torch.isfinite(out_host).all()
    assert float((out_host - exact).abs().max()) <= 2e-5 * max(1.0, float(exact.abs().max()))
    # a status left by a failed call does not poison the next one
    net._status.fill_(3)
    net.predict_host(X_host, R_host, out_host, tc=True)
    assert float((out_host - exact).abs().max()) <= 2e-5 * max(1.0, float(exact.abs().max()))


@pytest.mark.parametrize("I,pool,hidden,loss,rate,rc", [(1, "max", 0, "mse", None, False), (3, "all", 32, "nll", 0.3, False),
                                                        (2, "max", 32, "nll", None, True), (1, "avg", 0, "mse", 0.5, True)])
def test_input_gradients_match_the_oracle_chain(cuda, orc, I, pool, hidden, loss, rate, rc):
    """Z fed back as dZ = Z through the dense layers in test mode, pooling, rectifier and scan to dX."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m = 24
    p = synth.model_params(I, m, 19, pool, hidden=hidden)
    X, R = synth.ragged_batch(40, 25, 90, m, seed=20, n_frac=0.03, both_strands=rc)
    net = DeepBindNet(p, I, pool, loss=loss)
    if rate is not None:
        net.set_dropout(rate)
    Z, dX = net.input_gradients(torch.from_numpy(X).cuda(), torch.from_numpy(R.view(np.int32)).cuda(), strand_max=rc)
    wZ, wdX = orc.input_gradients({k: v.astype(np.float64) for k, v in p.items()}, X, R, pool, I, loss, strand_max=rc,
                                  dropout_rate=None if rate is None else np.full(I, rate))
    np.testing.assert_allclose(Z.cpu().numpy(), wZ, rtol=2e-5, atol=1e-6)
    assert np.abs(wdX).max() > 0
    assert np.max(np.abs(dX.cpu().numpy() - wdX)) <= 2e-5 * np.abs(wdX).max()


def test_gradient_maps_per_sequence(cuda, orc):
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import gradient_maps, predict
    rng = np.random.default_rng(5)
    m = 16
    seqs = seqs_of(rng, 70, 18, 60)
    p = synth.model_params(1, m, 21, "max")
    net = DeepBindNet(p, 1, "max", loss="mse")
    for rc in (False, True):
        Z, maps, strands = gradient_maps(net, seqs, reverse_complement=rc, batchsize=32)
        np.testing.assert_allclose(Z.cpu().numpy(), predict(net, seqs, reverse_complement=rc)["direct"].cpu().numpy(), rtol=1e-5, atol=1e-6)
        assert len(maps) == len(seqs) and all(g.shape == (len(s), 4) for g, s in zip(maps, seqs))
        assert (strands == 0).all() if not rc else set(strands.tolist()) <= {0, 1}
        Xo, Ro = orc.asbatch(seqs, m - 1, rc)
        _, wdX = orc.input_gradients(p, Xo, Ro, "max", 1, "mse", strand_max=rc)
        for b in (0, 13, 69):
            r = (2 * b + int(strands[b])) if rc else b
            want = wdX[Ro[r, 0] + m - 1:Ro[r, 1]]
            assert np.max(np.abs(maps[b] - want)) <= 2e-5 * max(np.abs(wdX).max(), 1e-12)


@pytest.mark.parametrize("rc", [False, True])
def test_mutation_maps(cuda, orc, rc):
    """Every single-base mutant scored through the device path against the oracle scoring the mutated strings."""
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import mutation_maps
    rng = np.random.default_rng(6)
    m, I = 16, 2
    seqs = seqs_of(rng, 4, 12, 30)
    p = synth.model_params(I, m, 23, "max")
    net = DeepBindNet(p, I, "max")
    Z, maps = mutation_maps(net, seqs, reverse_complement=rc)
    for b, s in enumerate(seqs):
        mutants = [s] + [s[:i] + c + s[i + 1:] for i in range(len(s)) for c in "ACGT"]
        want = orc.predict(p, mutants, m, "max", I, reverse_complement=rc)["direct"]
        z0, mt = want[0], want[1:].reshape(len(s), 4, I)
        d = (mt - z0) * np.maximum(0, np.sign(np.maximum(z0, mt)))
        np.testing.assert_allclose(Z[b], z0, rtol=1e-5, atol=1e-6)
        assert maps[b].shape == (len(s), 4, I)
        assert np.max(np.abs(maps[b] - d)) <= 1e-5 * max(np.abs(want).max(), 1e-6)
        # a mutation to the base already there changes nothing
        for i, c in enumerate(s):
            if c in "ACGT":
                assert np.all(maps[b][i, "ACGT".index(c)] == 0)
