"""Models instantiated from config text and trained by the sgd mirror, against the
CPU restatement of the same steps (forward, backward, L1 decay from
weight_decay_start on, dropout masks from supplied draws, Nesterov update)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ACGT = np.frombuffer(b"ACGT", dtype=np.uint8)

HIDDEN = """
return [motif_scan(num_motifs=16, motif_len=24, weight_decay=loguniform(1e-6,1e-3), init_scale=loguniform(1e-2,1e-1)),
        bias(), rectify(), allpool(), dropout(rate=choice([0.25, 0.5])),
        full(num_units=32, weight_decay=loguniform(1e-6,1e-3), init_scale=loguniform(1e-2,1e-1)), bias(), relu(),
        full(num_units=1, weight_decay=loguniform(1e-6,1e-3), init_scale=loguniform(1e-2,1e-1)), bias(), softmax()]
"""
LINEAR = """
return [motif_scan(num_motifs=16, motif_len=16, weight_decay=1e-4, init_scale=0.05), bias(), rectify(), maxpool(),
        full(num_units=1, weight_decay=1e-5, init_scale=0.05), bias()]
"""


def make_data(rng, n, L, classify):
    seqs = [ACGT[rng.integers(0, 4, L)].tobytes().decode() for _ in range(n)]
    Y = rng.integers(0, 2, size=(n, 1)).astype(np.float32) if classify else rng.standard_normal((n, 1)).astype(np.float32)
    return seqs, Y


def oracle_run(orc, net0, hp, seqs, Y, B, steps, start, drate, mrate, pool, I, loss, draws, rc=False):
    """The same training run on the CPU: returns the flat parameter vector."""
    P = orc.flatten(net0).astype(np.float32).copy()
    mom = np.zeros_like(P)
    m = net0["Wscan"].shape[0] // 4
    npool = 16 * (2 if pool == "all" else 1)
    nb = (len(seqs) + B - 1) // B
    for step in range(steps):
        lo = (step % nb) * B
        X, R = orc.asbatch(seqs[lo:lo + B], m - 1, rc)
        Yb = np.tile(np.repeat(Y[lo:lo + B], 2, axis=0) if rc else Y[lo:lo + B], (1, I))
        mask = None
        if draws is not None:
            U = draws[step][:len(R)]
            _, mask = orc.dropout_fp_tr(np.ones_like(U), hp["dropout"].astype(np.float32), U, matchrows=rc)
        decay = hp["decay"] if step >= start else None

        def grad(Pv):
            _, g = orc.train_grads(orc.unflatten(Pv, net0), X, R, Yb, pool, I, loss, mask, decay=decay, strand_pairs=rc)
            return orc.flatten(g)
        orc.nesterov_step(P, mom, drate, mrate, grad)
    return P


@pytest.mark.parametrize("text,I,classify,L,rc", [(HIDDEN, 3, True, 60, False), (LINEAR, 4, False, 40, False),
                                                  (HIDDEN, 2, True, 50, True)])
def test_training_run_matches_the_oracle(cuda, orc, text, I, classify, L, rc):
    import torch
    from deepbind_b200 import cfg
    from deepbind_b200.trainer import Trainer
    rng = np.random.default_rng(5)
    layers = cfg.loads(text)
    net, drawn = cfg.instantiate(layers, ninst=I, seed=11)
    plan = cfg.plan(layers)
    if plan.drop is not None:
        assert set(drawn) >= {"0.motif_scan.weight_decay", "0.motif_scan.init_scale", "4.dropout.rate"}
    seqs, Y = make_data(rng, 96, L, classify)
    B, steps, start = 32, 10, 4
    spec = cfg.sgd(rate=cfg.loguniform(0.005, 0.05), momentum=0.9, batchsize=B, max_epochs=100, max_steps=steps,
                   checkpoints=2, weight_decay_start=start)
    tr = Trainer(net, spec, seed=3)
    net0 = net.params_numpy()
    npool = 16 * (2 if plan.pool == "all" else 1)
    draws = rng.random((steps, B * (2 if rc else 1), npool * I)).astype(np.float32) if plan.drop is not None else None
    want = oracle_run(orc, net0, net.hparams, seqs, Y, B, steps, start, net.drate.cpu().numpy(), net.mrate.cpu().numpy(),
                      plan.pool, I, plan.loss, draws, rc)
    supply = (lambda step, shape: torch.from_numpy(draws[step][:shape[0]].copy()).cuda()) if draws is not None else None
    loss = tr.fit(seqs, Y, uniform_draws=supply, use_graph=False, reverse_complement=rc)
    got = net.P.cpu().numpy()
    scale = np.abs(want).max()
    assert np.max(np.abs(got - want)) <= 2e-5 * scale, (np.max(np.abs(got - want)), scale)
    assert np.all(np.isfinite(loss.cpu().numpy()))
    assert [s for s, _ in tr.history] == [5, 10] and all(h.shape == (I,) for _, h in tr.history)


@pytest.mark.parametrize("nseq", [128, 148])
def test_graph_replay_equals_eager_steps(cuda, nseq):
    """148 sequences: the fifth minibatch is short and runs call by call between the captured steps."""
    from deepbind_b200 import cfg
    from deepbind_b200.trainer import Trainer
    rng = np.random.default_rng(8)
    seqs, Y = make_data(rng, nseq, 40, False)
    spec = cfg.sgd(rate=0.02, momentum=0.9, batchsize=32, max_epochs=100, max_steps=12, checkpoints=1, weight_decay_start=5)
    out = []
    for use_graph, ministep in ((False, False), (True, False), (True, True), (True, True)):
        net, _ = cfg.instantiate(cfg.loads(LINEAR), ninst=5, seed=2)
        Trainer(net, spec, seed=1, ministep=ministep).fit(seqs, Y, use_graph=use_graph)
        out.append(net.P.cpu().numpy())
    np.testing.assert_array_equal(out[0], out[1])         # the operator-fused step, call by call and replayed
    # the two-launch step adds the samples' gradient shares in another order: same run up to rounding,
    # and the same bits every time
    assert np.max(np.abs(out[2] - out[0])) <= 2e-5 * np.abs(out[0]).max()
    np.testing.assert_array_equal(out[2], out[3])


def test_scoring_scales_by_one_minus_the_dropout_rate(cuda, orc):
    """Test mode of a dropout layer: Z = X * (1 - rate[model]) (elemwise.py:128-150)."""
    import torch
    from deepbind_b200 import cfg, synth
    net, _ = cfg.instantiate(cfg.loads(HIDDEN), ninst=3, seed=4)
    X, R = synth.uniform_batch(50, 60, 24, seed=1)
    dX = torch.from_numpy(X).cuda(); dR = torch.from_numpy(R.view(np.int32)).cuda()
    got = net.score(dX, dR).cpu().numpy()
    p = {k: v.astype(np.float64) for k, v in net.params_numpy().items()}
    keep = np.repeat(1.0 - net.hparams["dropout"], 32)
    p["W1"] = p["W1"] * keep[:, None]                 # scaling the pooled features = scaling the rows of W1
    want = orc.score_net(p, X, R, "all", 3)
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-6)
    assert net.dropout_rate is not None and np.all(net.hparams["dropout"] > 0)


@pytest.mark.parametrize("rc", [False, True])
def test_graph_training_with_device_drawn_dropout(cuda, rc):
    """Dropout under the captured step: the mask is drawn by a kernel of the graph (no draws supplied),
    the loss stays finite and falls on a learnable task, and the weights differ from a run without
    dropout."""
    from deepbind_b200 import cfg
    from deepbind_b200.trainer import Trainer
    rng = np.random.default_rng(11)
    seqs = [ACGT[rng.integers(0, 4, 50)].tobytes().decode() for _ in range(256)]
    Y = np.array([[1.0 if "ACGTAC" in s or "GGGG" in s else 0.0] for s in seqs], np.float32)
    spec = cfg.sgd(rate=0.05, momentum=0.9, batchsize=64, max_epochs=100, max_steps=60, checkpoints=3, weight_decay_start=1000)
    net, _ = cfg.instantiate(cfg.loads(HIDDEN), ninst=2, seed=3)
    t = Trainer(net, spec, seed=1)
    t.fit(seqs, Y, use_graph=True, reverse_complement=rc)
    losses = [h[1].cpu().numpy() if hasattr(h[1], "cpu") else np.asarray(h[1]) for h in t.history]
    assert len(losses) == 3 and all(np.isfinite(l).all() for l in losses)
    assert (losses[-1] < losses[0]).all()
    assert np.isfinite(net.P.cpu().numpy()).all()


def test_eight_step_replays_equal_eager_steps(cuda):
    """Enough minibatches for runs of eight steps per replay, cut by checkpoints, the start of the
    weight decay and the end of an epoch: same parameters and checkpoint losses as step-by-step calls."""
    from deepbind_b200 import cfg
    from deepbind_b200.trainer import Trainer
    rng = np.random.default_rng(9)
    seqs, Y = make_data(rng, 32 * 20 + 7, 40, False)               # 20 full minibatches and a short one
    spec = cfg.sgd(rate=0.02, momentum=0.9, batchsize=32, max_epochs=100, max_steps=75, checkpoints=3, weight_decay_start=11)
    out, hist = [], []
    for use_graph, ministep in ((False, False), (True, False), (True, True)):
        net, _ = cfg.instantiate(cfg.loads(LINEAR), ninst=3, seed=2)
        t = Trainer(net, spec, seed=1, ministep=ministep)
        t.fit(seqs, Y, use_graph=use_graph)
        out.append(net.P.cpu().numpy())
        hist.append([(s, np.asarray(l.cpu() if hasattr(l, "cpu") else l)) for s, l in t.history])
    np.testing.assert_array_equal(out[0], out[1])
    assert [s for s, _ in hist[0]] == [s for s, _ in hist[1]] == [s for s, _ in hist[2]] == [25, 50, 75]
    for (_, a), (_, b) in zip(hist[0], hist[1]):
        np.testing.assert_array_equal(a, b)
    # the two-launch step (replays of eight and of one, the short minibatch call by call in between):
    # the same run up to the order of the gradient sums
    assert np.max(np.abs(out[2] - out[0])) <= 5e-5 * np.abs(out[0]).max()
    for (_, a), (_, b) in zip(hist[0], hist[2]):
        np.testing.assert_allclose(a, b, rtol=1e-4)
