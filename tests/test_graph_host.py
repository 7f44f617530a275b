"""The node / plug engine on the host: pull evaluation, gradient accumulation over
fan-out, supernodes and chains, shape inference and the flag stacks, with small numeric
nodes written the way user code writes them against the reference's engine (no GPU)."""
import numpy as np
import pytest

from deepbind_b200 import cfg
from deepbind_b200 import graph as g


class scale_node(g.node):
    """Z = X * w"""

    def __init__(self, w):
        super(scale_node, self).__init__(["X"], ["Z"])
        self.w, self.nf, self.nb = w, 0, 0

    def _fprop(self, X):
        self.nf += 1
        return X * self.w

    def _bprop(self, dZ):
        self.nb += 1
        return dZ * self.w

    def _calc_shapes(self, X, Z):
        if X._shape:
            Z._shape = X._shape
        elif Z._shape:
            X._shape = Z._shape


class tanh_node(g.node):
    def __init__(self):
        super(tanh_node, self).__init__(["X"], ["Z"])

    def _fprop(self, X):
        return np.tanh(X)

    def _bprop(self, Z, dZ):
        return dZ * (1 - Z ** 2)

    def _calc_shapes(self, X, Z):
        if X._shape:
            Z._shape = X._shape


class add_node(g.node):
    def __init__(self):
        super(add_node, self).__init__(["A", "B"], ["Z"])

    def _fprop(self, A, B):
        return A + B

    def _bprop(self, dZ):
        return (dZ, dZ)

    def _calc_shapes(self, A, B, Z):
        Z._shape = A._shape or B._shape


def test_pull_evaluation_and_fanout_gradients():
    a, b, t, s = scale_node(2.0), scale_node(3.0), tanh_node(), add_node()
    # x -> a -> tanh -> s.A ; a -> b -> s.B : the output of a fans out to two consumers
    a >> t
    g.connect(t.Z, s.A)
    g.connect(a.Z, b.X)
    g.connect(b.Z, s.B)
    x = np.array([0.1, -0.2, 0.3])
    a.X.fpval = x
    z = s.Z.fpval
    np.testing.assert_allclose(z, np.tanh(2 * x) + 6 * x)
    assert a.nf == 1                                   # computed once, although two consumers pulled it
    s.Z.bpval = np.ones(3)
    dx = a.X.bpval
    np.testing.assert_allclose(dx, 2 * ((1 - np.tanh(2 * x) ** 2) + 3))   # both branches add up at a.Z
    assert a.nb == 1


def test_chain_and_supernode_export_unconnected_plugs():
    c = g.chain([scale_node(2.0), tanh_node(), scale_node(0.5)], name="net")
    assert [p.name for p in c.iplugs] == ["X"] and [p.name for p in c.oplugs] == ["Z"]
    out = c.eval(X=np.array([0.3]))
    np.testing.assert_allclose(out["Z"], 0.5 * np.tanh(0.6))
    assert c.X._fpval is g.plug_null                  # eval() leaves no values behind
    # two children with a plug of the same name: exported as A / B of the adder and X0, X1
    s1, s2, ad = scale_node(1.0), scale_node(1.0), add_node()
    g.connect(s1.Z, ad.A); g.connect(s2.Z, ad.B)
    sup = g.supernode([s1, s2, ad])
    assert [p.name for p in sup.iplugs] == ["X0", "X1"]
    assert sup.X0.origin() is s1.X and sup.Z.origin() is ad.Z
    assert sup.find("[2].Z") is ad.Z and sup.find(".X1") is sup.X1
    assert s1.path == "[0]" and ad.Z.path == "[2].Z"
    res = sup.eval(X0=np.array([1.0]), X1=np.array([2.0]))
    np.testing.assert_allclose(res["Z"], [3.0])


def test_flags_are_stacks():
    f = g.global_flags()
    assert "step" not in f and f.get("step", 7) == 7
    f.push("step", 1); f.push("step", 2)
    assert "step" in f and f["step"] == 2
    assert f.pop("step") == 2 and f.get("step") == 1
    f.pop("step")
    assert "step" not in f


def test_model_file_becomes_a_sequencenet_with_inferred_shapes():
    layers = cfg.loads("return [motif_scan(num_motifs=16, weight_decay=loguniform(1e-6, 1e-3)), bias(), rectify(), allpool(), "
                       "dropout(rate=choice([0.5, 0.75])), full(num_units=32), bias(), rectify(), full(num_units=1), bias(), softmax()]")
    m = g.from_layers(layers, motif_len=24)
    assert isinstance(m, g.sequencenet) and isinstance(m.conv_seq, g.chain) and isinstance(m.combiner, g.combine)
    assert [p.name for p in m.iplugs] == ["X_seq", "W0", "b", "R_seq", "F", "W1", "b0", "W2", "b1"]
    assert [p.name for p in m.oplugs] == ["cost0", "cost1", "cost2", "Z"]
    c = g.cost(m)
    assert isinstance(c.loss, g.nll)                  # a model ending in softmax trains with nll
    c.set_ninstance(3)
    c.F.shape = (None, 16)
    shapes = {p.name: p.shape for p in c.iplugs}
    assert shapes["W0"] == (96, 16) and shapes["b"] == (1, 16)
    assert shapes["W1"] == (48, 32)                   # 32 pooled features + the 16 feature columns of F
    assert shapes["W2"] == (32, 1) and shapes["b1"] == (1, 1) and shapes["Y"] == (None, 1)
    assert c.W1.origin().inst_axis == 0 and c.W0.origin().inst_axis == 1
    assert m.data_requirements() == {"target": "logistic", "padding": 23}
    assert all(n.ninst == 3 for n in m.conv_seq)
    # a layer list outside the DeepBind family: the fused-kernel peephole declines, the graph takes it
    odd = cfg.loads("return [motif_scan(num_motifs=8), bias(), rectify(), avgpool(), full(num_units=8), bias(), rectify(), "
                    "full(num_units=4), bias(), rectify(), full(num_units=1), bias()]")
    with pytest.raises(NotImplementedError):
        cfg.plan(odd)
    m2 = g.from_layers(odd, motif_len=12)
    c2 = g.cost(m2)
    assert isinstance(c2.loss, g.mse)
    c2.F.shape = (None, 16)
    names = [p.name for p in c2.iplugs]
    assert len(set(names)) == len(names)               # W, W beside the output net's W0, W1: numbered past them
    comb = [p for p in c2.iplugs if p.origin().node is m2.combiner][0]
    assert comb.shape == (8 + 16, 8)


def test_constraints_and_missing_gradient_are_reported():
    n = scale_node(1.0)
    with pytest.raises(AssertionError):
        n.Z.bpval                                      # an output nobody reads has no gradient unless one is set
    with pytest.raises(AssertionError):
        g.connect(n.X, scale_node(1.0).X)              # an input plug cannot feed another node's plug
