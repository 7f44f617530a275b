"""Models trained through the node / plug graph (every node one C-ABI operator) against the
fused kernels and against finite differences."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32


def planted(rng, n, L, motif="TGACGTCA"):
    seqs, y = [], []
    for i in range(n):
        s = "".join(rng.choice(list("ACGT"), size=L))
        if i % 2:
            p = int(rng.integers(0, L - len(motif)))
            s = s[:p] + motif + s[p + len(motif):]
        seqs.append(s); y.append(float(i % 2))
    return seqs, np.asarray(y, f32).reshape(-1, 1)


def batches_of(seqs, Y, B, pad, I, rc=False, with_regions=False):
    from deepbind_b200 import fused, smat as sm
    out = []
    for lo in range(0, len(seqs), B):
        X, R = fused.build_batch(seqs[lo:lo + B], pad, rc)
        Yb = np.tile(np.repeat(Y[lo:lo + B], 2, axis=0) if rc else Y[lo:lo + B], (1, I))
        b = {"X_seq": sm.sarray(X.view(-1, 1), np.uint8), "R_seq": sm.sarray(R, np.uint32),
             "F": sm.zeros((R.shape[0], 16), f32), "Y": sm.asarray(Yb)}
        if with_regions:
            b["regions"] = b["R_seq"]
        out.append((b, X, R, Yb))
    return out


def test_graph_and_fused_kernels_train_the_same_model(cuda):
    """The DeepBind family member of a model file, ten Nesterov steps from the same weights:
    through the graph (corr1ord, bias, relu, allpool, combine, ..., nll as separate
    operators) and through the fused scan and head kernels.  The graph's combiner also owns
    16 weight rows per model for the all-zero feature input F; they take no part in Z."""
    import torch
    from deepbind_b200 import cfg, graph as g, synth
    from deepbind_b200.model import DeepBindNet
    I, m, H = 2, 16, 8
    layers = cfg.loads("return [motif_scan(num_motifs=16), bias(), rectify(), allpool(), full(num_units=%d), bias(), rectify(), "
                       "full(num_units=1), bias(), softmax()]" % H)
    rng = np.random.default_rng(0)
    seqs, Y = planted(rng, 128, 40)
    spec = cfg.sgd(rate=0.05, momentum=0.9, batchsize=32, weight_decay_start=10 ** 9)
    tr = g.GraphTrainer(g.from_layers(layers, motif_len=m), spec, ninst=I, data_shapes={"X_seq": 1, "R_seq": 2, "F": 16}, seed=1)
    p = synth.model_params(I, m, 5, "all", hidden=H)
    p["Wscan"] *= 4; p["W1"] *= 8                        # large enough for visible learning in ten steps
    tr.param("W0").tensor.copy_(torch.from_numpy(p["Wscan"]))
    tr.param("b").tensor.copy_(torch.from_numpy(p["bscan"]).view(1, -1))
    W1g = tr.param("W1").tensor.view(I, 32 + 16, H)
    W1g[:, :32].copy_(torch.from_numpy(p["W1"]).view(I, 32, H))
    tr.param("b0").tensor.copy_(torch.from_numpy(p["b1"]).view(1, -1))
    tr.param("W2").tensor.copy_(torch.from_numpy(p["W2"]))
    tr.param("b1").tensor.copy_(torch.from_numpy(p["b2"]).view(1, -1))
    frows0 = W1g[:, 32:].clone()
    net = DeepBindNet(p, I, "all", loss="nll")
    net.set_rates(0.05, 0.9)
    bs = batches_of(seqs, Y, 32, m - 1, I)
    first = tr.loss([b for b, _, _, _ in bs])
    for step in range(10):
        b, X, R, Yb = bs[step % len(bs)]
        tr.train_step(b)
        net.train_step(X, R, torch.from_numpy(Yb).cuda())
    got = net.params_numpy("P")

    def close(a, w, name):
        assert np.max(np.abs(a - w)) <= 2e-5 * max(1e-3, np.abs(w).max()), name
    close(tr.param("W0").asnumpy(), got["Wscan"], "filters")
    close(tr.param("b").asnumpy().ravel(), got["bscan"].ravel(), "filter bias")
    close(W1g[:, :32].cpu().numpy().reshape(I * 32, H), got["W1"], "dense 1")
    close(tr.param("W2").asnumpy(), got["W2"], "dense 2")
    close(tr.param("b1").asnumpy().ravel(), got["b2"].ravel(), "output bias")
    assert torch.equal(W1g[:, 32:], frows0)              # no data gradient, no decay yet: the F rows stand still
    assert np.all(tr.loss([b for b, _, _, _ in bs]) < first)
    # predictions of the two paths agree
    Zg = tr.predict([bs[0][0]])
    Zf = torch.sigmoid(net.score(bs[0][1], bs[0][2])).cpu().numpy()
    np.testing.assert_allclose(Zg, Zf, rtol=2e-4, atol=2e-6)


def test_a_model_outside_the_family_trains_and_its_gradient_checks(cuda):
    """Three dense layers after mean pooling, mean squared error: the fused-kernel peephole
    declines it, the graph trains it; its gradient agrees with central differences."""
    from deepbind_b200 import cfg, graph as g
    layers = cfg.loads("return [motif_scan(num_motifs=8, init_scale=0.3, weight_decay=1e-3), bias(), rectify(), avgpool(), "
                       "full(num_units=8, init_scale=0.3, weight_decay=1e-3), bias(), rectify(), full(num_units=4, init_scale=0.3), bias(), "
                       "rectify(), full(num_units=1, init_scale=0.3), bias()]")
    with pytest.raises(NotImplementedError):
        cfg.plan(layers)
    I, m = 3, 8
    rng = np.random.default_rng(1)
    seqs, Y = planted(rng, 192, 30)
    spec = cfg.sgd(rate=cfg.loguniform(0.02, 0.05), momentum=0.9, batchsize=64, max_steps=150, max_epochs=100, checkpoints=3,
                   weight_decay_start=0)
    tr = g.GraphTrainer(g.from_layers(layers, motif_len=m), spec, ninst=I, data_shapes={"X_seq": 1, "R_seq": 2, "F": 16}, seed=4)
    bs = [b for b, _, _, _ in batches_of(seqs, Y, 64, m - 1, I)]
    assert g.gradcheck(tr, bs[0])
    first = tr.loss(bs)
    seen = []
    tr.fit(bs, on_checkpoint=lambda step, t: seen.append(step))
    assert seen == [50, 100, 150] and tr.step == 150
    last = tr.loss(bs)
    assert np.all(np.isfinite(last)) and np.all(last < 0.8 * first), (first, last)
    # device-side initialisation: per-model scale, zero-mean
    W = [t.P for t, q in zip(tr.trnodes, tr.tplugs) if isinstance(q.origin().node, g.full) and q.origin().node.size == 4][0].asnumpy()
    assert W.shape == (I * 8, 4)
    assert len({q.name for q in tr.tplugs}) == len(tr.tplugs)        # exported plug names are unique


def test_input_dropout_in_front_of_the_scan(cuda):
    """dropoutord before the scan, both strands: training drops bases (the reverse strand with the
    mirrored mask); scoring passes the sequence through and scales the scan by 1 - rate."""
    from deepbind_b200 import cfg, graph as g, smat as sm
    rate = 0.2
    nodes = [g.dropoutord(rate), g.motif_scan(8, motif_len=8, init_scale=0.3), g.bias(), g.rectify(), g.maxpool(),
             g.full(1, init_scale=0.3), g.bias(), g.softmax()]
    model = g.from_layers(nodes)
    spec = cfg.sgd(rate=0.05, momentum=0.9, batchsize=32, max_steps=40, max_epochs=100)
    tr = g.GraphTrainer(model, spec, ninst=1, data_shapes={"X_seq": 1, "R_seq": 2, "regions": 2, "F": 16}, seed=2)
    rng = np.random.default_rng(2)
    seqs, Y = planted(rng, 64, 30)
    bs = [b for b, _, _, _ in batches_of(seqs, Y, 32, 7, 1, rc=True, with_regions=True)]
    g.flags.push("reverse_complement", True)
    try:
        first = tr.loss(bs)
        # a training-mode pass drops bases pairwise-mirrored and never touches padding
        g.flags.push("train_mode", True)
        d = nodes[0]
        d.clear(); d.X.fpval = bs[0]["X_seq"]; d.regions.fpval = bs[0]["R_seq"]
        Z = d.Z.fpval.asnumpy().ravel(); X = bs[0]["X_seq"].asnumpy().ravel(); R = bs[0]["R_seq"].asnumpy()
        g.flags.pop("train_mode")
        d.clear(); d.X.fpval = g.plug_null; d.regions.fpval = g.plug_null
        assert np.all(Z[X == 255] == 255) and 0.1 < np.mean(Z[X < 4] == 254) < 0.3
        pad = 7
        for i in range(0, len(R), 2):
            (a, b), (c, e) = R[i], R[i + 1]
            assert np.array_equal(Z[c + pad:e] == 254, (Z[a + pad:b] == 254)[::-1])
        tr.fit(bs)
        assert np.all(tr.loss(bs) < first)
    finally:
        g.flags.pop("reverse_complement")
    # test mode: scan output scaled by 1 - rate
    scan = nodes[1]
    model.clear()
    out_with = tr.cost.eval_model(bs[:1])
    nodes[0].rate = 0.0
    out_without = tr.cost.eval_model(bs[:1])
    nodes[0].rate = rate
    assert not np.allclose(out_with, out_without)


def test_input_gradients_through_the_graph(cuda, orc):
    """eval(want_bprop_inputs=True): the output fed back as its own gradient reaches dX_seq [npos, 4],
    equal to what the operator chain of the composite net gives."""
    import torch
    from deepbind_b200 import cfg, graph as g, synth, smat as sm
    from deepbind_b200.model import DeepBindNet
    I, m = 1, 12
    layers = cfg.loads("return [motif_scan(num_motifs=16), bias(), rectify(), maxpool(), full(num_units=1), bias()]")
    model = g.from_layers(layers, motif_len=m)
    tr = g.GraphTrainer(model, cfg.sgd(), ninst=I, data_shapes={"X_seq": 1, "R_seq": 2, "F": 16}, seed=3)
    p = synth.model_params(I, m, 8, "max")
    p["Wscan"] *= 5
    assert [q.name for q in tr.tplugs] == ["W0", "b0", "W1", "b1"]      # two biases at the same level: b0 (scan), b1 (output)
    tr.param("W0").tensor.copy_(torch.from_numpy(p["Wscan"]))
    tr.param("b0").tensor.copy_(torch.from_numpy(p["bscan"]).view(1, -1))
    tr.param("W1").tensor.view(I, 32, 1)[:, :16].copy_(torch.from_numpy(p["W1"]).view(I, 16, 1))
    tr.param("b1").tensor.copy_(torch.from_numpy(p["b1"]).view(1, -1))
    X, R = synth.ragged_batch(20, 20, 50, m, seed=9)
    res = tr.cost.model.eval(X_seq=sm.asarray(X.reshape(-1, 1)), R_seq=sm.asarray(R), F=sm.zeros((20, 16), f32),
                             want_bprop_inputs=True)
    net = DeepBindNet(p, I, "max", loss="mse")
    Z, dX = net.input_gradients(torch.from_numpy(X).cuda(), torch.from_numpy(R.view(np.int32)).cuda())
    np.testing.assert_allclose(res["Z"].asnumpy(), Z.cpu().numpy(), rtol=1e-5, atol=1e-6)
    got = res["dX_seq"].asnumpy()
    assert got.shape == (X.size, 4) and np.abs(got).max() > 0
    assert np.max(np.abs(got - dX.cpu().numpy())) <= 2e-5 * np.abs(got).max()
