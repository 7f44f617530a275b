"""The two-launch minibatch step (db_ministep) against the operator-fused step
(DeepBindNet.train_step, itself checked against the CPU restatement in
test_gpu_trainer.py): same loss, gradient, parameters and momentum up to the order of the
gradient sums; bit-identical between eager launches and a CUDA-graph replay; walks a
device-resident dataset by its own step counter.  "Relative" = largest absolute
difference over the largest absolute value of the compared vector."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def _blocks(net, vec):
    return {k: getattr(net, vec)[int(net.offsets[i]):int(net.offsets[i + 1])] for i, k in enumerate(net.names)}


def _batch(kind, B, m, I, npool, seed, torch):
    from deepbind_b200 import synth
    g = synth.rng(seed)
    if kind == "uniform101":
        Xh, Rh = synth.uniform_batch(B, 101, m, seed=seed)
    elif kind == "uniform40":
        Xh, Rh = synth.uniform_batch(B, 40, m, seed=seed)
    else:                                   # ragged, with N bases; both strands when kind == "ragged_rc"
        Xh, Rh = synth.ragged_batch(B // 2 if kind == "ragged_rc" else B, 20, 90, m, seed, n_frac=0.05, both_strands=kind == "ragged_rc")
    X = torch.from_numpy(Xh).cuda(); R = torch.from_numpy(Rh.view(np.int32)).cuda()
    y = g.random((B // 2 if kind == "ragged_rc" else B, I)).astype(np.float32)
    if kind == "ragged_rc":
        y = np.repeat(y, 2, axis=0)
    mask = np.repeat(g.random((B // 2, npool * I)) >= 0.5, 2, axis=0) if kind == "ragged_rc" else g.random((B, npool * I)) >= 0.5
    return X, R, torch.from_numpy(y).cuda(), torch.from_numpy(mask).cuda()


CASES = [
    # I, pool, hidden, loss, batch kind, B, m, dropout, decay
    (1, "all", 32, "nll", "uniform101", 128, 24, True, False),
    (5, "max", 0, "mse", "uniform40", 64, 24, False, False),
    (3, "avg", 16, "mse", "ragged_rc", 64, 16, True, True),
    (2, "all", 0, "nll", "ragged", 50, 11, False, True),
    (4, "sum", 8, "mse", "ragged", 33, 24, True, False),
    # enough (sample, model) pairs for four samples per CTA
    (12, "max", 0, "mse", "uniform40", 64, 24, False, False),
    (10, "all", 8, "nll", "ragged_rc", 64, 16, True, True),
]


@pytest.mark.parametrize("I,pool,hidden,loss,kind,B,m,dropout,decay", CASES)
def test_one_step_equals_the_operator_fused_step(cuda, I, pool, hidden, loss, kind, B, m, dropout, decay):
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    npool = 16 * (2 if pool == "all" else 1)
    p = synth.model_params(I, m, 3, pool, hidden=hidden)
    X, R, Y, mask = _batch(kind, B, m, I, npool, 11, torch)
    if not dropout:
        mask = None
    rates = np.linspace(0.01, 0.03, I).astype(np.float32)

    def make():
        net = DeepBindNet(p, I, pool, loss=loss)
        net.set_rates(rates, 0.9)
        net.strand_pairs = kind == "ragged_rc"
        net.mP.copy_(torch.from_numpy(synth.rng(5).standard_normal(net.P.numel()).astype(np.float32) * 1e-3).cuda())
        if decay:
            net.set_decay({"Wscan": 1e-3, "W1": np.linspace(1e-4, 1e-3, I), "W2": 1e-3})
            net.decay_on = True
        return net
    old, new = make(), make()
    loss_old = old.train_step(X, R, Y, mask)
    ms = new.ministep(X, R, Y, mask)
    assert ms is not None
    ms.lookahead()
    loss_new = ms.run()
    torch.cuda.synchronize()
    assert int(ms.status.item()) == 0
    assert _rel(loss_new, loss_old) <= 2e-6
    for k, g_old in _blocks(old, "dP").items():
        assert _rel(_blocks(new, "dP")[k], g_old) <= 2e-5, k
    for vec in ("P", "mP"):
        for k, v_old in _blocks(old, vec).items():
            assert _rel(_blocks(new, vec)[k], v_old) <= 2e-6, (vec, k)
    # the look-ahead copy is the next step's starting point
    want = new.P + new.mrate * new.mP
    assert float((ms.PL - want).abs().max()) <= 1e-7 * float(want.abs().max())


@pytest.mark.parametrize("I,nmotif,pool,hidden,B,L,m", [
    (2, 32, "all", 16, 6, 30, 24),      # 32 filters per model: two groups of 16 in the scan, 64 pooled features
    (1, 16, "max", 128, 2, 1, 8),       # one-base sequences (rows = filter length), the widest hidden layer
    (3, 16, "avg", 0, 1, 200, 16),      # a single sample of 215 rows
])
def test_edge_shapes(cuda, I, nmotif, pool, hidden, B, L, m):
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    p = synth.model_params(I, m, 13, pool, hidden=hidden, nmotif=nmotif)
    Xh, Rh = synth.uniform_batch(B, L, m, seed=14)
    X = torch.from_numpy(Xh).cuda(); R = torch.from_numpy(Rh.view(np.int32)).cuda()
    Y = torch.from_numpy(synth.rng(15).standard_normal((B, I)).astype(np.float32)).cuda()

    def make():
        net = DeepBindNet(p, I, pool, loss="mse")
        net.set_rates(0.01, 0.9)
        return net
    old, new = make(), make()
    loss_old = old.train_step(X, R, Y)
    ms = new.ministep(X, R, Y)
    assert ms is not None
    ms.lookahead()
    loss_new = ms.run()
    torch.cuda.synchronize()
    assert int(ms.status.item()) == 0
    assert _rel(loss_new, loss_old) <= 2e-6
    for k, g_old in _blocks(old, "dP").items():
        assert _rel(_blocks(new, "dP")[k], g_old) <= 2e-5, k
    assert _rel(new.P, old.P) <= 2e-6


def test_steps_over_a_resident_dataset_eager_and_replayed(cuda):
    """Twelve steps over five stacked minibatches in a given order: graph replay equals
    eager launches bit for bit, both follow the operator-fused trainer step for step, and
    the counter ends at twelve."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    I, pool, hidden, m, B, nb = 2, "all", 32, 24, 64, 5
    p = synth.model_params(I, m, 4, pool, hidden=hidden)
    bs = [_batch("uniform40", B, m, I, 32, 20 + i, torch) for i in range(nb)]
    Xs, Rs, Ys, Ms = (torch.stack([b[k] for b in bs]) for k in range(4))
    order = torch.tensor([3, 0, 4, 1, 2], dtype=torch.int32, device="cuda")

    def make():
        net = DeepBindNet(p, I, pool, loss="nll"); net.set_rates([0.02, 0.01], [0.9, 0.8])
        return net
    old = make()
    for s in range(12):
        i = int(order[s % nb])
        old.train_step(Xs[i], Rs[i], Ys[i], Ms[i])
    eager = make()
    ms = eager.ministep(Xs, Rs, Ys, Ms, order=order)
    ms.lookahead()
    for s in range(12):
        ms.run()
    torch.cuda.synchronize()
    assert ms.counters.tolist()[0] == 12 and int(ms.status.item()) == 0
    for vec in ("P", "mP"):
        assert _rel(getattr(eager, vec), getattr(old, vec)) <= 2e-5
    replayed = make()
    ms2 = replayed.ministep(Xs, Rs, Ys, Ms, order=order)
    graph = ms2.capture(steps=4)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert ms2.counters.tolist()[0] == 12
    assert torch.equal(replayed.P, eager.P) and torch.equal(replayed.mP, eager.mP) and torch.equal(ms2.PL, ms.PL)
    assert torch.equal(ms2.loss, ms.loss)


def test_a_region_longer_than_announced_is_reported(cuda):
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    p = synth.model_params(1, 24, 3, "max")
    X, R, Y, _ = _batch("uniform40", 16, 24, 1, 16, 3, torch)
    net = DeepBindNet(p, 1, "max", loss="mse"); net.set_rates(0.01, 0.9)
    ms = net.ministep(X, R, Y, max_rows=40)          # the regions have 63 rows
    ms.lookahead(); ms.run()
    torch.cuda.synchronize()
    assert int(ms.status.item()) == 2
    ok = net.ministep(X, R, Y)
    ok.lookahead(); ok.run()
    torch.cuda.synchronize()
    assert int(ok.status.item()) == 0 and bool(torch.isfinite(net.P).all())


def test_unsupported_shapes_are_declined(cuda):
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    p = synth.model_params(1, 24, 3, "max", nmotif=8)
    X, R, Y, _ = _batch("uniform40", 16, 24, 1, 8, 3, torch)
    net = DeepBindNet(p, 1, "max", loss="mse")
    assert net.ministep(X, R, Y) is None             # 8 filters per model: outside the two-launch step
