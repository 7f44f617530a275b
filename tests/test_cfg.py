"""The config syntax of the reference's model / trainer files, executed against the
light-weight descriptors of deepbind_b200.cfg (no GPU needed)."""
import numpy as np
import pytest

MODEL = """
net = [
    motif_scan(num_motifs    = 16,
               motif_len     = 24,
               weight_decay  = loguniform(1e-15,1e-3),
               init_scale    = loguniform(1e-7,1e-3),
               ),
    bias(),
    rectify(),
    allpool(),
    dropout(rate = choice([0.0, 0.25, 0.5])),
    full(num_units = 32, weight_decay = loguniform(1e-10,1e-3), init_scale = loguniform(1e-5,1e-2)),
    bias(),
    relu(),
    full(num_units = 1, weight_decay = loguniform(1e-10,1e-3), init_scale = loguniform(1e-5,1e-2)),
    bias(),
    softmax(),
]

return net
"""

TRAINER = """
return sgd(rate = loguniform(0.0005,0.050), momentum = powuniform(0.95,0.99,0.5), batchsize = 64,
           max_epochs = 500, max_steps = 20000, checkpoints = 5, weight_decay_start = 100)
"""


def test_model_file_is_recognised():
    from deepbind_b200 import cfg
    layers = cfg.loads(MODEL)
    assert [type(l).__name__ for l in layers] == ["motif_scan", "bias", "rectify", "allpool", "dropout", "full", "bias", "relu",
                                                  "full", "bias", "softmax"]
    p = cfg.plan(layers)
    assert (p.pool, p.hidden, p.loss) == ("all", 32, "nll") and p.drop is layers[4]
    linear = cfg.loads("return [motif_scan(16, 16), bias(), rectify(), maxpool(), full(num_units=1), bias()]")
    q = cfg.plan(linear)
    assert (q.pool, q.hidden, q.loss, q.drop) == ("max", 0, "mse", None)


def test_unsupported_layer_lists_are_refused():
    from deepbind_b200 import cfg
    with pytest.raises(NotImplementedError):
        cfg.plan(cfg.loads("return [motif_scan(16, 16), rectify(), maxpool(), full(num_units=1), bias()]"))
    with pytest.raises(NotImplementedError):
        cfg.plan(cfg.loads("return [motif_scan(16, 16), bias(), rectify(), maxpool(), full(num_units=3), bias()]"))


def test_trainer_file_and_ranges():
    from deepbind_b200 import cfg
    t = cfg.loads(TRAINER)
    assert isinstance(t, cfg.sgd) and t.batchsize == 64 and t.weight_decay_start == 100 and t.checkpoints == 5
    rng = np.random.default_rng(0)
    r = t.rate.sample(rng, 1000)
    assert r.min() >= 0.0005 and r.max() < 0.05 and abs(np.median(np.log10(r)) - np.log10(0.005)) < 0.1
    mo = t.momentum.sample(rng, 1000)
    assert mo.min() >= 0.95 and mo.max() <= 0.99 and np.mean(mo) > 0.97        # sqrt skews towards the upper end
    c = cfg.choice([0.0, 0.25, 0.5]).sample(rng, 300)
    assert set(np.unique(c)) == {0.0, 0.25, 0.5}
    u = cfg.uniform(2, 3).sample(rng, 100)
    assert u.min() >= 2 and u.max() < 3
    assert cfg.fixed([1, 2]).sample(rng, 2).tolist() == [1, 2]


def test_named_variables_instead_of_return():
    from deepbind_b200 import cfg
    a, b = cfg.loads("x = bias()\ny = sgd(rate=0.1)\n", "x", "y")
    assert isinstance(a, cfg.bias) and b.rate == 0.1
