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


def test_minibatch_feed_walks_the_dataset(cuda):
    """db_minibatch_fetch: minibatch order[step % nbatch] of three arrays per launch, the step
    counter kept on the device; odd sizes take the byte path."""
    import torch
    from deepbind_b200 import fused
    g = torch.Generator(device="cuda").manual_seed(1)
    nbatch = 5
    A = torch.randint(0, 255, (nbatch, 1003), dtype=torch.uint8, device="cuda", generator=g)
    B = torch.randn((nbatch, 64, 3), device="cuda", generator=g)
    C = torch.rand((nbatch, 64, 32), device="cuda", generator=g) >= 0.5
    a, b, c = torch.empty_like(A[0]), torch.empty_like(B[0]), torch.empty_like(C[0])
    feed = fused.MinibatchFeed([(A, a), (B, b), (C, c)])
    for step in range(12):
        feed.fetch()
        i = step % nbatch
        assert torch.equal(a, A[i]) and torch.equal(b, B[i]) and torch.equal(c, C[i])
    assert feed.counters.tolist() == [12, 0]
    order = torch.tensor([3, 0, 4, 1, 2], dtype=torch.int32, device="cuda")
    feed = fused.MinibatchFeed([(B, b)], order=order)
    for step in range(7):
        feed.fetch()
        assert torch.equal(b, B[int(order[step % nbatch])])
    big = torch.randn((3, 1 << 20), device="cuda", generator=g)        # several CTAs per launch
    dst = torch.empty_like(big[0])
    feed = fused.MinibatchFeed([(big, dst)])
    for step in range(4):
        feed.fetch()
        assert torch.equal(dst, big[step % 3])


def test_graph_with_feed_equals_eager_steps_over_the_dataset(cuda):
    """fetch + step replayed from one graph = eager steps on the same minibatches in order."""
    import torch
    from deepbind_b200 import fused, synth
    from deepbind_b200.model import DeepBindNet
    m, B, I, nbatch = 24, 32, 4, 3
    p = synth.model_params(I, m, 3, "max")
    Xh, Rh = synth.uniform_batch(B * nbatch, 40, m, seed=1)
    rows = B * (40 + m - 1)
    Xall = torch.from_numpy(np.stack([np.concatenate([Xh[i * rows:(i + 1) * rows], np.full(m - 1, 255, np.uint8)])
                                      for i in range(nbatch)])).cuda()
    R = torch.from_numpy(Rh[:B].view(np.int32)).cuda()
    Yall = torch.from_numpy(synth.rng(2).standard_normal((nbatch, B, I)).astype(np.float32)).cuda()
    eager = DeepBindNet(p, I, "max", loss="mse"); eager.set_rates(0.02, 0.9)
    for s in range(7):
        eager.train_step(Xall[s % nbatch], R, Yall[s % nbatch])
    net = DeepBindNet(p, I, "max", loss="mse"); net.set_rates(0.02, 0.9)
    P0, m0 = net.P.clone(), net.mP.clone()
    Xs, Ys = Xall[0].clone(), Yall[0].clone()
    feed = fused.MinibatchFeed([(Xall, Xs), (Yall, Ys)])
    graph, _ = net.capture_train_step(Xs, R, Ys, feed=feed)
    net.P.copy_(P0); net.mP.copy_(m0)
    for _ in range(7):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(net.P, eager.P) and torch.equal(net.mP, eager.mP)


@pytest.mark.parametrize("matchrows", [0, 1])
def test_device_drawn_dropout_masks(cuda, matchrows):
    """db_dropout_mask: keep-rate 1 - rate[model] per model block, a fresh draw on every launch (also
    when the launch is replayed from a CUDA graph), strand pairs sharing their row when asked."""
    import torch
    from deepbind_b200 import _lib
    from deepbind_b200.smat import bind_stream
    dll = _lib.load()
    nrow, k, I = 512, 32, 3
    rate = torch.tensor([0.5, 0.2, 0.0], dtype=torch.float32, device="cuda")
    M = torch.zeros((nrow, k * I), dtype=torch.bool, device="cuda")
    counters = torch.zeros(2, dtype=torch.int32, device="cuda")

    def draw():
        bind_stream()
        dll.db_dropout_mask(M.data_ptr(), nrow, k * I, rate.data_ptr(), I, matchrows, counters.data_ptr())
    draw()
    first = M.clone()
    keep = first.float().view(nrow, I, k).mean(dim=(0, 2)).cpu().numpy()
    assert abs(keep[0] - 0.5) < 0.03 and abs(keep[1] - 0.8) < 0.03 and keep[2] == 1.0
    if matchrows:
        assert torch.equal(first[0::2], first[1::2])
    else:
        assert not torch.equal(first[0::2], first[1::2])
    draw()
    assert not torch.equal(M, first) and counters.tolist() == [2, 0]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        draw()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        draw()
    seen = []
    for _ in range(3):
        g.replay(); torch.cuda.synchronize()
        seen.append(M.clone())
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])
    assert counters.tolist() == [6, 0]


def test_several_steps_per_graph_equal_single_steps(cuda):
    """Four steps captured into one graph and replayed twice = eight eager steps over the dataset."""
    import torch
    from deepbind_b200 import fused, synth
    from deepbind_b200.model import DeepBindNet
    m, B, I, nbatch = 24, 32, 2, 3
    p = synth.model_params(I, m, 3, "all", hidden=32)
    Xh, Rh = synth.uniform_batch(B * nbatch, 40, m, seed=1)
    rows = B * (40 + m - 1)
    Xall = torch.from_numpy(np.stack([np.concatenate([Xh[i * rows:(i + 1) * rows], np.full(m - 1, 255, np.uint8)])
                                      for i in range(nbatch)])).cuda()
    R = torch.from_numpy(Rh[:B].view(np.int32)).cuda()
    g = synth.rng(2)
    Yall = torch.from_numpy(np.tile(g.integers(0, 2, size=(nbatch, B, 1)).astype(np.float32), (1, 1, I))).cuda()
    Mall = torch.from_numpy(g.random((nbatch, B, 32 * I)) >= 0.5).cuda()
    eager = DeepBindNet(p, I, "all", loss="nll"); eager.set_rates(0.02, 0.9)
    for s in range(8):
        eager.train_step(Xall[s % nbatch], R, Yall[s % nbatch], Mall[s % nbatch])
    net = DeepBindNet(p, I, "all", loss="nll"); net.set_rates(0.02, 0.9)
    P0, m0 = net.P.clone(), net.mP.clone()
    Xs, Ys, Ms = Xall[0].clone(), Yall[0].clone(), Mall[0].clone()
    feed = fused.MinibatchFeed([(Xall, Xs), (Yall, Ys), (Mall, Ms)])
    graph, _ = net.capture_train_step(Xs, R, Ys, Ms, feed=feed, steps=4)
    net.P.copy_(P0); net.mP.copy_(m0)
    graph.replay(); graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(net.P, eager.P) and torch.equal(net.mP, eager.mP)
    assert feed.counters.tolist() == [8, 0]


def test_graph_survives_scratch_growth(cuda):
    """A captured step keeps the scratch address it saw.  A later, larger call makes the
    library take a bigger scratch buffer; the old one must stay alive, so replaying the
    small graph afterwards still gives the eager result.  Growing inside a capture is refused."""
    import torch
    from deepbind_b200 import _lib, synth, SmatException
    from deepbind_b200.model import DeepBindNet
    dll = _lib.load()
    m, B, I = 24, 64, 1
    p = synth.model_params(I, m, 3, "all", hidden=32)
    Xh, Rh = synth.uniform_batch(B, 60, m, seed=1)
    g = synth.rng(2)
    X = torch.from_numpy(Xh).cuda(); R = torch.from_numpy(Rh.view(np.int32)).cuda()
    Y = torch.from_numpy(g.integers(0, 2, (B, I)).astype(np.float32)).cuda()
    eager = DeepBindNet(p, I, "all", loss="nll"); eager.set_rates(0.02, 0.9)
    for _ in range(3):
        eager.train_step(X, R, Y)
    net = DeepBindNet(p, I, "all", loss="nll"); net.set_rates(0.02, 0.9)
    P0, m0 = net.P.clone(), net.mP.clone()
    graph, _ = net.capture_train_step(X, R, Y)
    net.P.copy_(P0); net.mP.copy_(m0)
    graph.replay()
    # a later call needs more scratch than anything so far (whatever earlier tests of this
    # process left): the library moves to a larger buffer, which a column sum then uses
    before = dll.db_scratch_bytes()
    dll.db_reserve_scratch(2 * before + (4 << 20))
    big = torch.ones((1_000_000, 64), dtype=torch.float32, device="cuda")
    s = torch.empty(64, dtype=torch.float32, device="cuda")
    dll.db_colsum(s.data_ptr(), big.data_ptr(), big.shape[0], 64)
    torch.cuda.synchronize()
    assert dll.db_scratch_bytes() > before and float(s[0]) == 1_000_000.0
    del big
    junk = torch.full((before // 4 + 1024,), float("nan"), device="cuda")      # would land on a freed scratch buffer
    graph.replay(); graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(net.P, eager.P) and torch.equal(net.mP, eager.mP)
    del junk
    # growth while capturing is an error, not an allocation
    need = dll.db_scratch_bytes() * 4
    from deepbind_b200.smat import bind_stream
    cg = torch.cuda.CUDAGraph()
    msg = None
    with torch.cuda.graph(cg):
        bind_stream()
        try:
            dll.db_reserve_scratch(need)
        except SmatException as e:
            msg = str(e)
    bind_stream()
    assert msg is not None and "being captured" in msg
    dll.db_reserve_scratch(need)
    assert dll.db_scratch_bytes() >= need
