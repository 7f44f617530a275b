"""A training step replayed from a CUDA graph gives the same parameters, bit for
bit, as the same steps launched one call at a time."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("I,pool,hidden,loss", [(1, "all", 32, "nll"), (5, "max", 0, "mse")])
def test_graph_replay_equals_eager_steps(cuda, I, pool, hidden, loss):
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, B = 24, 64
    p = synth.model_params(I, m, 3, pool, hidden=hidden)
    Xh, Rh = synth.uniform_batch(B, 60, m, seed=1)
    g = synth.rng(2)
    X = torch.from_numpy(Xh).cuda(); R = torch.from_numpy(Rh.view(np.int32)).cuda()
    Y = torch.from_numpy(np.tile(g.standard_normal((B, 1)).astype(np.float32), (1, I))).cuda()
    npool = 16 * (2 if pool == "all" else 1)
    mask = torch.from_numpy(g.random((B, npool * I)) >= 0.5).cuda()

    eager = DeepBindNet(p, I, pool, loss=loss); eager.set_rates(0.02, 0.9)
    for _ in range(4):
        eager.train_step(X, R, Y, mask)

    net = DeepBindNet(p, I, pool, loss=loss); net.set_rates(0.02, 0.9)
    P0, m0 = net.P.clone(), net.mP.clone()
    graph, loss_t = net.capture_train_step(X, R, Y, mask)
    net.P.copy_(P0); net.mP.copy_(m0)              # the warm-up steps moved the parameters
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(net.P, eager.P) and torch.equal(net.mP, eager.mP)
    assert np.all(np.isfinite(loss_t.cpu().numpy()))


@pytest.mark.parametrize("strand_max", [False, True])
def test_captured_scoring_equals_direct_scoring(cuda, strand_max):
    """score() replayed from a CUDA graph, also after its input buffers were refilled in place."""
    import torch
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    m, n = 24, 96
    p = synth.model_params(3, m, 5, "max")
    net = DeepBindNet(p, 3, "max")
    Xa, Ra = synth.uniform_batch(n, 40, m, seed=6)
    Xb, _ = synth.uniform_batch(n, 40, m, seed=7)
    X = torch.from_numpy(Xa).cuda(); R = torch.from_numpy(Ra.view(np.int32)).cuda()
    graph, out = net.capture_score(X, R, strand_max)
    graph.replay()
    assert torch.equal(out, net.score(X, R, strand_max))
    X.copy_(torch.from_numpy(Xb).cuda())
    graph.replay()
    assert torch.equal(out, net.score(X, R, strand_max))
    assert out.shape == ((n // 2 if strand_max else n), 3)
