"""Dependency-graph model engine with the semantics of ``deepity``'s node / plug graph,
and the DeepBind layer nodes on top of the library's drop-in operators.

The reference builds every model as a graph of *nodes* joined by *plugs* and evaluates it
by pull: asking an output plug for its value runs ``fprop`` of the node behind it, which
asks its input plugs, and so on; asking an input plug for its gradient runs ``bprop`` the
same way (code/libs/deepity/deepity/plug.py:45-140, node.py:47-338).  A *supernode* wraps
a sub-graph and re-exports its unconnected plugs (node.py:365-460); ``chain`` connects
nodes in sequence (std/chain.py:38-51); trainable weights enter through ``trainable``
nodes bound to slices of one flat parameter vector (std/trainable.py:38-65,
sgd.py:287-354).  This module restates that engine for Python 3 with the same names and
call conventions, so that user code written against it (``class mynode(node)`` with
``_fprop(self, X)`` / ``_bprop(self, Z, dZ)``, ``a >> b``, ``model.eval(X=...)``) runs,
and provides the nodes the DeepBind models use:

    corr1ord / motif_scan, maxpool / avgpool / allpool, dropoutord   (kangaroo/_ext/*.py)
    bias, relu / rectify, linear, logistic, dropout, full, combine   (deepity/std/*.py)
    softmax, mse, nll, costsum, sequencenet, trainer cost wrapper    (std/softmax.py, loss.py,
                                                                      trainer.py, kangaroo/model.py)

Every node computes through the C ABI of libdeepbind_b200.so (``api_corr1ord``,
``api_poolrgn``, ``api_blockwise_dot*``, ``api_dropout_*``, ``api_gradstep*``, ``db_*``);
PyTorch only owns the memory.  :func:`from_layers` turns the layer list of a model file
into a ``sequencenet`` as the reference's loader does (_io_/load.py:51-76);
:func:`deepbind_b200.cfg.plan` is the peephole that replaces the whole graph of the
DeepBind family by the fused kernels, and anything else trains through this graph with
:class:`GraphTrainer`.
"""
import inspect
import re

import numpy as np
import torch

from . import _lib, cfg
from . import deepity_smat as dsm
from . import kangaroo_smat as ks
from . import smat as sm
from .smat import sarray


# ------------------------------------------------------------------------ flags
class global_flags(object):
    """Named stacks of values steering evaluation (deepity/globals.py:43-76):
    ``train_mode``, ``bprop_mode``, ``want_bprop_inputs``, ``reverse_complement``,
    ``step``, ``weight_decay_start``.  A flag is "in" the set while its stack is non-empty."""

    def __init__(self):
        self._stacks = {}

    def __contains__(self, name):
        return bool(self._stacks.get(name))

    def get(self, name, default_value=None):
        st = self._stacks.get(name)
        return st[-1] if st else default_value

    __getitem__ = get

    def push(self, name, value=True):
        self._stacks.setdefault(name, []).append(value)

    def pop(self, name):
        st = self._stacks[name]
        value = st.pop()
        if not st:
            del self._stacks[name]
        return value


flags = global_flags()


# ------------------------------------------------------------------ small helpers
def _dll():
    dll = _lib.load()
    sm.bind_stream()
    return dll


def _f32(t):
    return sarray(t.contiguous(), np.float32)


def _add(a, b):
    """Sum of two plug values (device arrays, numbers, or None = nothing)."""
    if a is None:
        return b
    if b is None:
        return a
    if isinstance(b, sarray) and not isinstance(a, sarray):
        a, b = b, a
    if isinstance(a, sarray):
        other = b.tensor if isinstance(b, sarray) else torch.as_tensor(np.asarray(b, np.float32), device=a.tensor.device)
        return sarray((a.tensor + other).contiguous(), a.dtype)
    return a + b


class _plug_null(object):
    """'No value yet' (distinct from None, which is a legitimate value)."""

    def __bool__(self):
        return False

    def __repr__(self):
        return "plug_null"


plug_null = _plug_null()


# ------------------------------------------------------------------------- plugs
class plug(object):
    """One named input or output of a node.  ``srcs`` feed it, ``dsts`` read it; its
    forward value is pulled from the sources (summed if several), its backward value from
    the destinations (plug.py:112-140).  ``shape`` is (rows, cols) per model instance with
    None for a free dimension; ``inst_axis`` says which axis grows with the number of
    instances (columns, except weights of dense layers: rows)."""

    def __init__(self, owner, name):
        self.node, self.name = owner, name
        self.srcs, self.dsts = [], []
        self._fpval = self._bpval = plug_null
        self._shape = None
        self.inst_axis = 1
        self.trainable = True

    def has_src(self):
        return bool(self.srcs)

    def has_dst(self):
        return bool(self.dsts)

    def is_iplug(self):
        return any(p is self for p in self.node.iplugs)

    def is_oplug(self):
        return any(p is self for p in self.node.oplugs)

    def has_upstream(self):
        """Is there anything upstream that computes (rather than merely holds) a value?"""
        if not self.srcs:
            return self.is_oplug()
        return any(s.has_upstream() for s in self.srcs)

    @property
    def path(self):
        return self.node.path + "." + self.name

    def rename(self, newname):
        del self.node.__dict__[self.name]
        self.name = newname
        self.node.__dict__[newname] = self

    def origin(self):
        """The plug of an ordinary node that a supernode's plug stands for."""
        if not isinstance(self.node, supernode):
            return self
        return self.dsts[0].origin() if self.is_iplug() else self.srcs[0].origin()

    # -- values
    @property
    def fpval(self):
        if self._fpval is plug_null:
            if self.srcs:
                total = plug_null
                for src in self.srcs:
                    total = src.fpval if total is plug_null else _add(total, src.fpval)
                self._fpval = total
            elif self.is_oplug():
                self.node.fprop()
            else:
                self._fpval = None
        return self._fpval

    @fpval.setter
    def fpval(self, value):
        self._fpval = value

    @property
    def bpval(self):
        if self._bpval is plug_null:
            if self.dsts:
                total = plug_null
                for dst in self.dsts:
                    total = dst.bpval if total is plug_null else _add(total, dst.bpval)
                self._bpval = total
            elif self.is_iplug():
                self.node.bprop()
            else:
                raise AssertionError("output plug %s has no destination and no gradient was set on it" % self.path)
        return self._bpval

    @bpval.setter
    def bpval(self, value):
        assert not self.dsts, "cannot set a gradient on a plug with a downstream connection"
        self._bpval = value

    # -- shapes
    @property
    def shape(self):
        if self._shape is None:
            self._calc_shape([])
        return self._shape

    @shape.setter
    def shape(self, shape):
        self._shape = shape

    def _calc_shape(self, visited):
        if self._shape is not None:
            return True
        if any(v is self for v in visited):
            return False
        for p in self.srcs + self.dsts:             # connected plugs carry the same value
            if p._calc_shape(visited + [self]):
                self._shape = p._shape
                return True
        self.node.calc_shapes(visited + [self])     # else the owner may deduce it from its other plugs
        return self._shape is not None

    def _check(self):
        if isinstance(self.node, supernode):
            assert not (self.is_iplug() and len(self.dsts) > 1), "a supernode's input plug feeds one inner plug"
            assert not (self.is_oplug() and len(self.srcs) > 1), "a supernode's output plug has one inner source"
        else:
            assert not (self.is_iplug() and self.dsts), "a node's input plug cannot feed another plug"
            assert not (self.is_oplug() and self.srcs), "a node's output plug cannot have a source"

    def __rshift__(self, other):
        connect(self, other); return other

    def __lshift__(self, other):
        connect(other, self); return self

    def __repr__(self):
        return "<plug %s>" % self.path


def connect(src, dst):
    """src >> dst.  A node stands for its first output (as src) or first input (as dst)."""
    if isinstance(src, node):
        src = src.oplugs[0]
    if isinstance(dst, node):
        dst = dst.iplugs[0]
    assert isinstance(src, plug) and isinstance(dst, plug), "connect() takes plugs or nodes"
    src.dsts.append(dst); dst.srcs.append(src)
    src._check(); dst._check()


def disconnect(src, dst):
    if isinstance(src, node):
        src = src.oplugs[0]
    if isinstance(dst, node):
        dst = dst.iplugs[0]
    src.dsts = [p for p in src.dsts if p is not dst]
    dst.srcs = [p for p in dst.srcs if p is not src]


# ------------------------------------------------------------------------- nodes
def _argnames(fn):
    return [n for n in inspect.signature(fn).parameters]


class node(object):
    """A vertex of the graph.  Subclasses name their plugs and write ``_fprop`` (returns
    the output values from the input values named by its arguments) and ``_bprop``
    (returns the input gradients; an argument ``dZ`` receives the gradient of output Z,
    any other name the forward value of that plug), plus ``_calc_shapes`` for shape
    inference (node.py:47-338)."""

    def __init__(self, iplugs, oplugs, name=None):
        self.name, self.ninst, self._parent = name, 1, None
        self.iplugs = [plug(self, n) for n in iplugs]
        self.oplugs = [plug(self, n) for n in oplugs]
        for p in self.iplugs + self.oplugs:
            self.__dict__[p.name] = p

    parent = property(lambda self: self._parent)

    @property
    def path(self):
        if self._parent is None:
            return ""
        for i, child in enumerate(self._parent):
            if child is self:
                rel = "[%d]" % i
                for nm, attr in self._parent.__dict__.items():
                    if attr is self:
                        rel = "." + nm
                        break
                return self._parent.path + rel
        return ""

    # -- traversal
    def _visit(self, path, callback):
        callback(path, self)
        for nm, attr in list(self.__dict__.items()):
            if isinstance(attr, (plug, cfg.paramdef)):
                new = callback(path + "." + nm, attr)
                if new is not None:
                    setattr(self, nm, new)

    def visit(self, callback):
        """callback(path, obj) for this node, its plugs and hyper-parameters and, for a
        supernode, everything inside it."""
        self._visit("", callback)

    def set_ninstance(self, ninst):
        def fn(path, obj):
            if isinstance(obj, node):
                obj.ninst = ninst
        self.visit(fn)

    def find(self, path):
        if path == "":
            return self
        assert path.startswith(".")
        return getattr(self, path[1:])

    def requirements(self):
        reqs = {}

        def fn(path, obj):
            if isinstance(obj, node):
                reqs.update({path + "." + k: v for k, v in obj._requirements().items()})
        self.visit(fn)
        return reqs

    def _requirements(self):
        return {}

    def data_requirements(self):
        reqs = self.requirements()
        padding = max([0] + [v for k, v in reqs.items() if k.endswith("sequence_padding")])
        target = [v for k, v in reqs.items() if k.endswith("target")]
        assert len(target) <= 1
        return {"target": target[0] if target else [], "padding": padding}

    # -- shapes
    def calc_shapes(self, visited):
        if any(v is self for v in visited):
            return
        args = {n: getattr(self, n) for n in _argnames(self._calc_shapes)}
        for p in args.values():                     # what the neighbours know about these plugs comes first
            p._calc_shape(visited + [self])
        self._calc_shapes(**args)

    def _calc_shapes(self):
        raise NotImplementedError("%s does not implement _calc_shapes" % type(self).__name__)

    # -- evaluation
    def clear(self):
        """Forgets every computed value; values set by hand on unconnected input plugs stay."""
        def fn(path, obj):
            if isinstance(obj, plug):
                if obj.has_src() or obj.is_oplug():
                    obj._fpval = plug_null
                obj._bpval = plug_null
        self.visit(fn)

    def fprop(self):
        for p in self.oplugs:
            assert p._fpval is plug_null, "fprop needs undefined outputs (call clear())"
        inputs = {}
        for n in _argnames(self._fprop):
            p = getattr(self, n)
            assert any(q is p for q in self.iplugs), "_fprop may only ask for input plugs (got %s)" % n
            inputs[n] = p.fpval
        out = self._fprop(**inputs)
        if not isinstance(out, tuple):
            out = (out,)
        for p, v in zip(self.oplugs, out):
            p._fpval = v

    def bprop(self):
        for p in self.iplugs:
            assert p._bpval is plug_null, "bprop needs undefined input gradients (call clear())"
        inputs = {}
        for n in _argnames(self._bprop):
            if n.startswith("d") and hasattr(self, n[1:]) and isinstance(getattr(self, n[1:]), plug):
                p = getattr(self, n[1:])
                assert any(q is p for q in self.oplugs), "_bprop may only ask for gradients of output plugs (got %s)" % n
                inputs[n] = p.bpval
            else:
                inputs[n] = getattr(self, n).fpval
        out = self._bprop(**inputs)
        if not isinstance(out, tuple):
            out = (out,)
        for p, v in zip(self.iplugs, out):
            p._bpval = v

    def _fprop(self):
        raise NotImplementedError("cannot propagate through %s" % type(self).__name__)

    def _bprop(self):
        raise NotImplementedError("cannot back-propagate through %s" % type(self).__name__)

    def eval(self, clear=True, want_bprop_inputs=False, bprop_inputs_loss=None, **inputs):
        """Sets the given input plugs, pulls every output plug and returns {name: value}.
        With ``want_bprop_inputs`` the output Z is fed back as its own gradient (through
        ``bprop_inputs_loss``, a loss node, without the minibatch mean) and the gradients
        of the given inputs are returned as ``d<name>`` (node.py:288-338)."""
        self.clear()
        flags.push("want_bprop_inputs", want_bprop_inputs)
        flags.push("bprop_mode", want_bprop_inputs)
        try:
            for k, v in inputs.items():
                getattr(self, k).fpval = v
            result = {p.name: p.fpval for p in self.oplugs}
            if want_bprop_inputs:
                for p in self.oplugs:
                    if p.name == "Z":
                        loss = bprop_inputs_loss or mse()
                        loss.ninst = self.ninst
                        loss.batchmean = False
                        loss.clear()
                        loss.Z.fpval = result["Z"]
                        loss.Y.fpval = sm.zeros_like(result["Z"])
                        loss.Ymask.fpval = None
                        g = loss.Z.bpval
                        result["Zmask"] = loss.Zmask._fpval if loss.Zmask._fpval is not plug_null else None
                        ncol = g.shape[1] // max(1, self.ninst)
                        if ncol > 1:                                   # only target 0 of each model is fed back
                            t = g.tensor.view(g.shape[0], self.ninst, ncol).clone()
                            t[:, :, 1:] = 0
                            g = _f32(t.view(g.shape))
                        p._bpval = g
                    else:
                        p._bpval = None
                result.update({"d" + p.name: p.bpval for p in self.iplugs if p.name in inputs})
        finally:
            flags.pop("want_bprop_inputs")
            flags.pop("bprop_mode")
        if clear:
            self.clear()
        for k in inputs:
            getattr(self, k).fpval = plug_null
        return result

    def __rshift__(self, other):
        connect(self, other); return other

    def __lshift__(self, other):
        connect(other, self); return self


class supernode(node):
    """A sub-graph behind one interface: every inner plug left unconnected becomes a plug
    of the supernode (same name; R, R -> R0, R1 when names collide)."""

    def __init__(self, children, name=None):
        self._children = list(children)
        for c in self._children:
            c._parent = self
        inner_in = [p for c in self._children for p in c.iplugs if not p.has_src()]
        inner_out = [p for c in self._children for p in c.oplugs if not p.has_dst()]
        super(supernode, self).__init__(self._names(inner_in), self._names(inner_out), name)
        for outer, inner in zip(self.iplugs, inner_in):
            connect(outer, inner); outer.inst_axis = inner.inst_axis
        for inner, outer in zip(inner_out, self.oplugs):
            connect(inner, outer); outer.inst_axis = inner.inst_axis

    @staticmethod
    def _names(plugs):
        raw = [p.name for p in plugs]
        keep = {n for n in raw if raw.count(n) == 1}       # names that are unique stay as they are
        out = []
        for i, nm in enumerate(raw):
            if nm not in keep:                             # R, R -> R0, R1 (skipping numbers already in use)
                k = raw[:i].count(nm)
                while nm + str(k) in keep or nm + str(k) in out:
                    k += 1
                nm = nm + str(k)
            out.append(nm)
        return out

    def _visit(self, path, callback):
        super(supernode, self)._visit(path, callback)
        for i, child in enumerate(self._children):
            rel = "[%d]" % i
            for nm, attr in self.__dict__.items():
                if attr is child:
                    rel = "." + nm
                    break
            child._visit(path + rel, callback)

    def find(self, path):
        if path == "":
            return self
        m = re.match(r"^\[(\d+)\](.*)", path)
        if m:
            return self._children[int(m.group(1))].find(m.group(2))
        m = re.match(r"^\.(\w+)$", path)
        if m:
            return getattr(self, m.group(1))
        m = re.match(r"^\.(\w+)(.+)", path)
        return getattr(self, m.group(1)).find(m.group(2))

    def __iter__(self):
        return iter(self._children)

    def __getitem__(self, i):
        return self._children[i]

    def __len__(self):
        return len(self._children)

    def calc_shapes(self, visited):
        return

    def fprop(self):
        return

    def bprop(self):
        return


class chain(supernode):
    """Nodes connected one after the other; what stays unconnected is exported."""

    def __init__(self, children, name=None):
        for a, b in zip(children[:-1], children[1:]):
            connect(a, b)
        super(chain, self).__init__(children, name)


class trainable(node):
    """Feeds a slice P of the flat parameter vector into a weight plug and receives the
    gradient into the matching slice dP (std/trainable.py:38-65)."""

    def __init__(self, P, dP=None):
        super(trainable, self).__init__([], ["Z"])
        self.P, self.dP = P, dP

    def _fprop(self):
        return self.P

    def bprop(self):
        g = self.Z.bpval
        if g is None:
            self.dP.tensor.zero_()
        elif isinstance(g, sarray):
            self.dP.tensor.copy_(g.tensor.view(self.dP.tensor.shape))
        else:
            self.dP.tensor.fill_(float(g))
        self.Z._bpval = plug_null

    def enforce_constraints(self):
        owner = self.Z.dsts[0].origin().node
        if hasattr(owner, "enforce_constraints"):
            owner.enforce_constraints(self.P)

    def _calc_shapes(self, Z):
        pass


# ------------------------------------------------------------- element-wise nodes
class elemwise(node):
    def _calc_shapes(self, X, Z):
        if X._shape:
            Z._shape = X._shape
        elif Z._shape:
            X._shape = Z._shape


class linear(elemwise):
    """Z = X"""

    def __init__(self):
        super(linear, self).__init__(["X"], ["Z"])

    def _fprop(self, X):
        return X

    def _bprop(self, dZ):
        return dZ


class relu(elemwise):
    """Z = max(0, X); dX = dZ * sign(Z)   (std/elemwise.py:71-78)"""

    def __init__(self):
        super(relu, self).__init__(["X"], ["Z"])

    def _fprop(self, X):
        if X is None or "disable_relu" in flags:
            return X
        Z = sm.empty_like(X)
        _dll().db_relu(Z.data_ptr(), X.data_ptr(), X.size)
        return Z

    def _bprop(self, dZ, Z):
        if dZ is None:
            return None
        dX = sm.empty_like(dZ)
        _dll().db_relu_bprop(dX.data_ptr(), dZ.data_ptr(), Z.data_ptr(), Z.size)
        return dX


class rectify(relu):
    pass


class logistic(elemwise):
    def __init__(self):
        super(logistic, self).__init__(["X"], ["Z"])

    def _fprop(self, X):
        if X is None:
            return None
        Z = sm.empty_like(X)
        _dll().db_logistic(Z.data_ptr(), X.data_ptr(), X.size)
        return Z

    def _bprop(self, dZ, Z):
        return None if dZ is None else _f32(dZ.tensor * (Z.tensor - Z.tensor * Z.tensor))


class dropout(elemwise):
    """Training: Z = X * M with M ~ Bernoulli(1 - rate) per model, one mask per strand pair
    with ``reverse_complement``; otherwise Z = X * (1 - rate)   (std/elemwise.py:116-157)."""

    def __init__(self, rate=0.5, activerange=None):
        super(dropout, self).__init__(["X"], ["Z"])
        self.M, self.rate, self.activerange = None, rate, activerange

    def _rate(self, X):
        if not isinstance(self.rate, sarray):
            r = np.asarray(self.rate, np.float32).ravel()
            self.rate = sm.asarray(np.broadcast_to(r, (self.ninst,)).copy() if r.size == 1 else r, np.float32)
        return self.rate

    def _fprop(self, X):
        if X is None:
            return None
        if np.isscalar(self.rate) and self.rate == 0:
            return X
        rate = self._rate(X)
        if "train_mode" in flags:
            Z, self.M = dsm.dropout_fp_train(X, rate, "reverse_complement" in flags)
            return Z
        return dsm.dropout_fp_test(X, rate)

    def _bprop(self, dZ):
        if dZ is None or (np.isscalar(self.rate) and self.rate == 0):
            return dZ
        if "train_mode" in flags:
            dX = dsm.dropout_bp_tr(dZ, self.M)
            self.M = None
            return dX
        return dsm.dropout_bp_te(dZ, self.rate)


class bias(elemwise):
    """Z = X + b (row broadcast); db = column sums of dZ (+ negdecay), zero before
    ``start_training``   (std/elemwise.py:162-180)."""

    def __init__(self, init=0.0, init_mu=0, negdecay=None, viz=True, start_training=0):
        super(bias, self).__init__(["X", "b"], ["Z"])
        self.init, self.init_mu, self.viz = init, init_mu, viz
        self.negdecay, self.start_training = negdecay, start_training

    def _fprop(self, X, b):
        if X is None:
            return None
        Z = sm.empty_like(X)
        _dll().db_bias_add(Z.data_ptr(), X.data_ptr(), b.data_ptr(), X.shape[0], X.shape[1])
        return Z

    def _bprop(self, dZ):
        if dZ is None:
            return (None, 0)
        db = sm.empty((1, dZ.shape[1]), np.float32)
        _dll().db_colsum(db.data_ptr(), dZ.data_ptr(), dZ.shape[0], dZ.shape[1])
        if self.negdecay:
            db.tensor.add_(float(self.negdecay))
        if self.start_training > flags.get("step", 0):
            db.tensor.zero_()
        return (dZ, db)

    def _calc_shapes(self, X, Z, b):
        if X._shape and b._shape:
            assert X._shape[1] == b._shape[1]
        elif X._shape:
            b._shape = (1, X._shape[1])
        elif b._shape:
            X._shape = (None, b._shape[1])
        elemwise._calc_shapes(self, X, Z)


# ------------------------------------------------------------------- dense layers
def _decay_of(owner, W):
    """Per-model L1 decay as a device vector, or None."""
    d = owner.decay
    if d is None:
        return None
    if not isinstance(d, sarray):
        v = np.asarray(d, np.float32).ravel()
        owner.decay = d = sm.asarray(np.broadcast_to(v, (owner.ninst,)).copy() if v.size == 1 else v, np.float32)
    return d


def _decay_active():
    return flags.get("weight_decay_start", 0) <= flags.get("step", 0)


def _l1_cost(owner, W, per_column):
    """decay[inst] * sum |W_inst| as [1, ninst], or 0 (full.py:91-109, corr1ord.py:112-115)."""
    d = _decay_of(owner, W)
    if d is None or "bprop_mode" in flags or not _decay_active():
        return 0
    a = W.tensor.abs()
    if per_column:                                          # instances side by side on columns
        c = a.sum(dim=0).view(owner.ninst, -1).sum(dim=1)
    else:                                                   # instances stacked on rows
        c = a.reshape(owner.ninst, -1).sum(dim=1)
    return _f32((c * d.tensor.view(-1)).view(1, -1))


def _l1_grad(owner, W, dW, k):
    """dW += decay[inst] * sign(W): madd_bcast(sign(W), decay, k, dW) (full.py:111-119)."""
    d = _decay_of(owner, W)
    if d is None or dW is None or not _decay_active():
        return
    dsm.madd_bcast(_f32(torch.sign(W.tensor)), d, k, dW)


class full(node):
    """Z = X . W per model (weights of the models stacked on rows), cost = decay * sum|W|
    (std/full.py:41-129)."""

    def __init__(self, num_units, weight_decay=None, init_scale=None, init_bias=None, ishape=None, oshape=None):
        super(full, self).__init__(["X", "W"], ["Z", "cost"])
        self.size = num_units
        self.init = init_scale if init_scale is not None else 0.001
        self.init_mu = init_bias if init_bias is not None else 0.0
        self.decay = weight_decay
        self.ishape, self.oshape = ishape, oshape
        self.W.inst_axis = 0

    def _fprop(self, X, W):
        if X is None:
            return (None, 0)
        return (dsm.blockwise_dot(X, W, self.ninst), _l1_cost(self, W, per_column=False))

    def _bprop(self, X, W, dZ):
        want = "want_bprop_inputs" in flags
        dX = dsm.blockwise_dot_nt(dZ, W, self.ninst) if (self.X.has_upstream() or want) else None
        dW = dsm.blockwise_dot_tn(X, dZ, self.ninst, W) if (self.W.has_upstream() or want) else None
        _l1_grad(self, W, dW, W.size // self.ninst)
        return (dX, dW)

    def _calc_shapes(self, X, W, Z):
        if X._shape and W._shape:
            assert X._shape[1] == W._shape[0]
        elif X._shape:
            W._shape = (X._shape[1], self.size)
        elif W._shape:
            X._shape = (None, W._shape[0])
        Z._shape = (None, self.size)


class combine(full):
    """A dense layer over the logical concatenation of inputs X0..Xk, block by block
    without stacking them; an input with one model's columns is shared by all models
    (std/full.py:131-196)."""

    def __init__(self, num_inputs, size, decay=None, init=None, init_mu=None, start_training=None, ishape=None, oshape=None):
        node.__init__(self, ["X%d" % i for i in range(num_inputs)] + ["W"], ["Z", "cost"])
        self.num_inputs, self.size = num_inputs, size
        self.init = init if init is not None else 0.001
        self.init_mu = init_mu if init_mu is not None else 0.0
        self.decay, self.start_training = decay, start_training
        self.ishape, self.oshape = ishape, oshape
        self.W.inst_axis = 0

    def _inputs(self):
        X = [p.fpval for p in self.iplugs[:self.num_inputs]]
        bc = [self.ninst > 1 and (X[t].shape[1] == self.iplugs[t].shape[1] if X[t] is not None else True) for t in range(len(X))]
        return X, bc

    def _fprop(self, W):
        X, bc = self._inputs()
        return (dsm.blockwise_dot_combined(X, W, self.ninst, bc), _l1_cost(self, W, per_column=False))

    def _bprop(self, W, dZ):
        X, bc = self._inputs()
        mask = None
        if self.start_training:
            assert len(X) == len(self.start_training)
            mask = [s < flags.get("step", 0) for s in self.start_training]
        dX = dsm.blockwise_dot_nt_combined(X, dZ, W, self.ninst, bc)
        dW = dsm.blockwise_dot_tn_combined(X, dZ, W, self.ninst, bc, mask)
        _l1_grad(self, W, dW, W.size // self.ninst)
        return tuple(dX) + (dW,)

    def _calc_shapes(self, W, Z):
        total = 0
        for X in self.iplugs[:self.num_inputs]:
            assert X.srcs, "%s has no source; its width cannot be determined" % X.name
            X.srcs[0]._calc_shape([self])
            X._shape = X.srcs[0]._shape or (None, 0)
            total += X._shape[1]
        if W._shape:
            assert total == W._shape[0]
        else:
            W._shape = (total, self.size)
        Z._shape = (None, self.size)


class softmax(node):
    """One column per model: the logistic function; gradients pass unchanged, the loss
    node's dZ = Z - Y already being the gradient with respect to the pre-activation
    (std/softmax.py:50-77)."""

    def __init__(self, ngroup=1):
        super(softmax, self).__init__(["X"], ["Z"])
        self.ngroup = ngroup

    def _fprop(self, X):
        if X is None or flags.get("disable_softmax", False):
            return X
        nchunk = self.ngroup * self.ninst
        Z = sm.empty_like(X)
        if nchunk == X.shape[1]:
            _dll().db_logistic(Z.data_ptr(), X.data_ptr(), X.size)
            return Z
        A = X.tensor.reshape(-1, X.shape[1] // nchunk) if nchunk > 1 else X.tensor
        return _f32(torch.softmax(A, dim=1).reshape(X.shape))

    def _bprop(self, dZ):
        return dZ

    def _requirements(self):
        return {"target": "logistic"}

    def _calc_shapes(self, X, Z):
        if X._shape:
            Z._shape = X._shape
        elif Z._shape:
            X._shape = Z._shape


# ------------------------------------------------------------------------ losses
class loss_node(node):
    """Per-model loss of predictions Z against targets Y (std/loss.py:40-139): elementwise
    loss, masked by Ymask and by Zmask (the stronger strand of each pair with
    ``reverse_complement``), mean over ALL rows, summed over a model's outputs, scaled.
    Backward: dZ = (Z - Y) masked the same way, times 1/rows."""
    kind = None

    def __init__(self, ngroup=1):
        super(loss_node, self).__init__(["Z", "Y", "Ymask"], ["loss", "Zmask"])
        self.ngroup = ngroup
        self.Y.trainable = False
        self.Ymask.trainable = False
        self.batchmean = True

    def _zmask(self, Z):
        if "reverse_complement" not in flags:
            return None
        M = sm.zeros(Z.shape, np.bool_)
        dsm.calc_Zmask(Z, M)
        return M

    def _run(self, Z, Y, Ymask, Zmask, want_dz):
        n, c = Z.shape
        lo = sm.empty((1, c), np.float32)
        dz = sm.empty_like(Z) if want_dz else None
        _dll().db_loss(self.kind, Z.data_ptr(), Y.data_ptr(), Ymask.data_ptr() if Ymask is not None else None,
                       Zmask.data_ptr() if Zmask is not None else None, n, c, lo.data_ptr(),
                       dz.data_ptr() if dz is not None else None)
        return lo, dz

    def _fprop(self, Z, Y, Ymask):
        assert self.ngroup == 1, "grouped losses are not implemented (nor are they in the reference)"
        Zmask = self._zmask(Z)
        lo, _ = self._run(Z, Y, Ymask, Zmask, False)
        per_model = lo.tensor.view(self.ninst, -1).sum(dim=1).view(1, -1)       # sum over a model's outputs
        return (_f32(per_model), Zmask)

    def _bprop(self, Z, Y, Ymask):
        Zmask = self._zmask(Z)
        self.Zmask._fpval = Zmask
        _, dz = self._run(Z, Y, Ymask, Zmask, True)                             # (Z - Y) masked, / rows
        if not self.batchmean:
            dz.tensor.mul_(float(Z.shape[0]))
        return dz

    def _calc_shapes(self, Z, Y, loss):
        if Z._shape and Y._shape:
            assert Z._shape[1] == Y._shape[1]
        elif Z._shape:
            Y._shape = (None, Z._shape[1])
        elif Y._shape:
            Z._shape = (None, Y._shape[1])
        loss._shape = (1, 1)


class mse(loss_node):
    """0.5 * mean (Z - Y)^2"""
    kind = 0


class nll(loss_node):
    """-mean [ Y log max(1e-15, Z) + (1 - Y) log max(1e-15, 1 - Z) ]"""
    kind = 1


class costsum(node):
    """Sums whatever is connected to X (the plug adds its sources); gradient 1 to each."""

    def __init__(self):
        super(costsum, self).__init__(["X"], ["cost"])

    def _fprop(self, X):
        return X

    def _bprop(self):
        return 1

    def _calc_shapes(self, cost):
        cost._shape = (1, 1)


# ---------------------------------------------------------------- sequence nodes
class corr1ord(node):
    """Motif scan of an ordinal sequence: Z [npos, nfilter*ninst] = corr1ord(W, X); cost =
    L1 decay; filter gradient, and the input gradient when ``want_bprop_inputs`` is set
    (kangaroo/_ext/corr1ord.py:42-158).  With an input-dropout node upstream the test-mode
    output is scaled by 1 - rate."""

    def __init__(self, nfilter, fsize=None, decay=0, init=1e-3, nchannel=4, name=None, constraint=None, start_training=0):
        super(corr1ord, self).__init__(["X", "W"], ["Z", "cost"], name)
        self.nfilter, self.fsize, self.decay, self.init = nfilter, fsize, decay, init
        self.nchannel, self.constraint, self.start_training = nchannel, constraint, start_training

    def enforce_constraints(self, W):
        """pfm / psam: every position's four weights are log-probabilities normalised by
        their sum / maximum; (lo, hi): clipping (corr1ord.py:60-78)."""
        if self.constraint is None:
            return
        t = W.tensor
        if self.constraint in ("pfm", "psam"):
            F = torch.exp(t).view(-1, self.nchannel, t.shape[1])
            norm = F.sum(dim=1, keepdim=True) if self.constraint == "pfm" else F.max(dim=1, keepdim=True)[0]
            t.copy_(torch.log(F / norm).view(t.shape))
        elif isinstance(self.constraint, tuple):
            lo, hi = self.constraint
            t.clamp_(min=lo, max=hi)
        else:
            raise NotImplementedError("constraint %r" % (self.constraint,))

    def _fprop(self, X, W):
        Z = sm.zeros((X.shape[0], W.shape[1]), W.dtype)
        ks.corr1ord(W, X, Z, self.nchannel)
        if "train_mode" not in flags and self.X.srcs:
            up = self.X.srcs[0].origin().node if isinstance(self.X.srcs[0].node, supernode) else self.X.srcs[0].node
            if isinstance(up, dropoutord) and up.rate > 0:
                Z.tensor.mul_(1.0 - float(up.rate))
        return (Z, _l1_cost(self, W, per_column=True))

    def _bprop(self, X, W, dZ):
        dW = sm.zeros_like(W)
        ks.corr1ord_bprop_W(dW, X, dZ, self.nchannel)
        _l1_grad(self, W, dW, max(1, W.shape[0] // self.ninst))      # k = rows / ninst, as corr1ord.py:126 passes it
        dX = None
        if "want_bprop_inputs" in flags:
            dX = sm.zeros((X.size, 4), W.dtype)
            ks.corr1ord_bprop_X(dX, W, dZ, self.nchannel)
        if self.start_training > flags.get("step", 0):
            dW.tensor.zero_()
        return (dX, dW)

    def _requirements(self):
        assert self.fsize is not None, "set corr1ord.fsize before anything that needs shapes"
        return {"sequence_padding": self.fsize - 1}

    def _calc_shapes(self, X, W, Z):
        assert self.fsize is not None, "set corr1ord.fsize before anything that needs shapes"
        if not X._shape:
            X._shape = (None, 1)
        if not W._shape:
            W._shape = (self.fsize * self.nchannel, self.nfilter)
        Z._shape = (None, self.nfilter)


class motif_scan(corr1ord):
    def __init__(self, num_motifs, motif_len=None, weight_decay=0, init_scale=1e-3):
        super(motif_scan, self).__init__(nfilter=num_motifs, fsize=motif_len or num_motifs, decay=weight_decay, init=init_scale)


class _pool(node):
    ptype, ncolmul = None, 1

    def __init__(self, regions=None):
        super(_pool, self).__init__(["X", "R"], ["Z"])
        self.I = None
        self.regions = regions or [(0, None)]

    def _fprop(self, X, R):
        Z, self.I = ks.poolrgn(X, R, ptype=self.ptype, want_argmax=self.ptype != "avg" and "bprop_mode" in flags)
        return Z

    def _bprop(self, X, R, dZ):
        dX = sm.zeros_like(X)
        ks.poolrgn_bprop(dX, R, dZ, self.I, ptype=self.ptype)
        self.I = None
        return (dX, None)

    def _calc_shapes(self, X, R, Z):
        k = self.ncolmul
        if X._shape and Z._shape:
            assert k * X._shape[1] == Z._shape[1]
        elif X._shape:
            Z._shape = (None, k * X._shape[1])
        elif Z._shape:
            X._shape = (None, Z._shape[1] // k)

    def _requirements(self):
        return {"sequence_pooling": self.regions}


class maxpool(_pool):
    """Z[i, j] = max over the rows of region i (kangaroo/_ext/poolrgn.py:40-95)."""
    ptype = "max"


class avgpool(_pool):
    """Z[i, j] = mean over the rows of region i (poolrgn.py:105-133)."""
    ptype = "avg"


class allpool(_pool):
    """Z[i, 2j] = max, Z[i, 2j+1] = mean (poolrgn.py:135-198)."""
    ptype, ncolmul = "all", 2


class dropoutord(elemwise):
    """Dropout on the ordinal input: a dropped base becomes 254 (contributes nothing to the
    scan); padding is never dropped; with ``reverse_complement`` the reverse strand of a
    pair gets the forward strand's mask mirrored (kangaroo/_ext/dropoutord.py:41-76).
    Test mode passes X through; the scan then scales by 1 - rate."""

    def __init__(self, rate):
        node.__init__(self, ["X", "regions"], ["Z"])
        self.rate, self.M = rate, None

    def _fprop(self, X, regions):
        if X is None or "train_mode" not in flags:
            return X
        Z, self.M = ks.dropoutord_fp_train(X, float(self.rate))
        if "reverse_complement" in flags:
            M = self.M.tensor.view(-1).clone()
            R = regions.asnumpy().astype(np.int64)
            pad = M.numel() - int(R[-1, -1])
            for i in range(0, len(R), 2):
                a, b = R[i]; c, d = R[i + 1]
                M[c + pad:d] = torch.flip(M[a + pad:b], dims=[0])
            Zt = X.tensor.view(-1).clone()
            Zt[~M] = 254
            self.M = sarray(M.view(-1, 1), np.bool_)
            Z = sarray(Zt.view(-1, 1), np.uint8)
        return Z

    def _bprop(self, dZ):
        self.M = None
        return (dZ, None)


class sequencenet(supernode):
    """convnet(s) over the sequence input(s) and a feature vector F, joined by a
    ``combine`` layer whose output feeds ``outputnet`` (kangaroo/model.py:45-132):

        X_seq, R_seq -- convnet --+-- combiner -- outputnet -> Z
        F ---------- featurenet --+
    """

    def __init__(self, convnets, outputnet, combiner_size=None, combiner_decay=None, combiner_init=None,
                 combiner_init_mu=None, combiner_start=None):
        if not combiner_size:
            combiner_size = sum(c.Z.shape[1] for c in convnets)
        self.combiner = combine(len(convnets) + 1, size=combiner_size, ishape=(1, -1), decay=combiner_decay,
                                init=combiner_init, init_mu=combiner_init_mu, start_training=combiner_start)
        self.outputnet = outputnet
        connect(self.combiner.Z, outputnet.X)
        for i, c in enumerate(convnets):
            self.__dict__["conv" + ("_" + c.name if c.name else str(i))] = c
            connect(c.Z, getattr(self.combiner, "X%d" % i))
        self.featurenet = linear()
        connect(self.featurenet.Z, getattr(self.combiner, "X%d" % len(convnets)))
        super(sequencenet, self).__init__(list(convnets) + [self.featurenet, self.combiner, self.outputnet])
        for i, c in enumerate(convnets):
            Xp = getattr(self, "X%d" % i)
            Rp = getattr(self, "R%d" % i, None) or getattr(self, "R")
            Xp.rename("X_%s" % c.name if c.name else "X%d" % i)
            Rp.rename("R_%s" % c.name if c.name else "R%d" % i)
        getattr(self, "X%d" % len(convnets)).rename("F")


_NODE_OF = {"motif_scan": motif_scan, "bias": bias, "relu": relu, "rectify": rectify, "maxpool": maxpool, "avgpool": avgpool,
            "allpool": allpool, "dropout": dropout, "full": full, "softmax": softmax, "logistic": logistic}


def from_layers(layers, motif_len=None):
    """The graph of a model file's layer list, as the reference's loader builds it
    (_io_/load.py:51-76): everything before the first ``full`` becomes the convnet "seq",
    that ``full`` becomes the combiner (which also takes the feature input F), the rest
    the output net.  ``layers`` are :mod:`deepbind_b200.cfg` descriptors or nodes of this
    module; ``motif_len`` sets the filter length as the training scripts set ``fsize``."""
    nodes = []
    for l in layers:
        if isinstance(l, node):
            nodes.append(l)
            continue
        nm = type(l).__name__
        if nm not in _NODE_OF:
            raise NotImplementedError("no node for layer %r" % nm)
        kw = dict(vars(l))
        if nm == "dropout":
            kw = {"rate": kw["rate"]}
        if nm == "full":
            kw = {"num_units": kw["num_units"], "weight_decay": kw["weight_decay"], "init_scale": kw["init_scale"], "init_bias": kw["init_bias"]}
        nodes.append(_NODE_OF[nm](**kw))
    first_full = next(i for i, n in enumerate(nodes) if isinstance(n, full))
    for n in nodes[:first_full]:
        if isinstance(n, corr1ord) and motif_len:
            n.fsize = motif_len
    conv = chain(nodes[:first_full], name="seq")
    comb = nodes[first_full]
    out = chain(nodes[first_full + 1:])
    return sequencenet([conv], out, combiner_size=comb.size, combiner_decay=comb.decay, combiner_init=comb.init)


# ------------------------------------------------------------------------ training
class cost(supernode):
    """model -> loss -> costsum, with every ``cost`` output of the model added in
    (deepity/trainer.py:52-76): ``nll`` when the model ends in a softmax, else ``mse``."""

    def __init__(self, model, lossfunc=None):
        self.model = model
        self.costsum = costsum()
        self.loss = nll() if isinstance(model.Z.origin().node, softmax) else mse()
        connect(model.Z, self.loss.Z)
        connect(self.loss.loss, self.costsum.X)
        for p in model.oplugs:
            if p.name.startswith("cost"):
                connect(p, self.costsum.X)
        super(cost, self).__init__([model, self.loss, self.costsum])

    def _set(self, batch):
        for k, v in batch.items():
            if hasattr(self, k):
                getattr(self, k).fpval = v

    def _unset(self, batch):
        self.clear()
        for k in batch:
            if hasattr(self, k):
                getattr(self, k).fpval = None

    def eval_loss(self, batches):
        total = None
        for batch in batches:
            self._set(batch)
            l = self.loss.loss.fpval.asnumpy().ravel()
            total = l if total is None else total + l
            self._unset(batch)
        return total / max(1, len(batches))

    def eval_model(self, batches):
        out = []
        for batch in batches:
            self._set(batch)
            out.append(self.model.Z.fpval.asnumpy())
            self._unset(batch)
        return np.vstack(out)

    def bprop_trainable(self, trnodes, batch):
        """One gradient evaluation: the gradient 1 enters at the summed cost and every
        trainable node pulls its own (trainer.py:142-160)."""
        self._set(batch)
        self.cost.bpval = 1
        flags.push("bprop_mode", True)
        try:
            for t in trnodes:
                t.bprop()
        finally:
            flags.pop("bprop_mode")
        self._unset(batch)


class GraphTrainer(object):
    """Nesterov / momentum SGD over a node graph with the bookkeeping of ``deepity.sgd``
    (sgd.py:87-163,287-354): one flat vector each for parameters, gradient, momentum and
    per-element rates; every trainable plug (an unconnected input plug that is not a data
    input) gets a ``trainable`` node bound to its slice; parameters start as
    randn * init[instance] + init_mu, drawn on the device; a step is
    ``gradstep(P, dP, drate, mP, mrate, grad=bprop_trainable, nesterov)``."""

    def __init__(self, model, spec=None, ninst=1, data_shapes=None, seed=0):
        self.spec = spec or cfg.sgd()
        self.model = model
        self.cost = cost(model)
        self.cost.set_ninstance(ninst)
        self.ninst = ninst
        data_shapes = dict(data_shapes or {})
        for k, ncol in data_shapes.items():
            if hasattr(self.cost, k):
                getattr(self.cost, k).shape = (None, ncol)
        self.data_names = set(data_shapes) | {"Y", "Ymask"}
        rng = np.random.default_rng(seed)

        def sample(path, obj):                      # one draw per model instance for every hyper-parameter range
            if isinstance(obj, cfg.paramdef):
                return np.asarray(obj.sample(rng, ninst))
        self.cost.visit(sample)
        self.tplugs = [p for p in self.cost.iplugs
                       if p.origin().trainable and p.name not in self.data_names and p.shape]
        self.rate = np.broadcast_to(np.asarray(self._draw(self.spec.rate, rng), np.float32), (ninst,)).copy()
        self.momentum = np.broadcast_to(np.asarray(self._draw(self.spec.momentum, rng), np.float32), (ninst,)).copy()
        self._setup(seed)
        self.step = 0

    def _draw(self, v, rng):
        return v.sample(rng, self.ninst) if isinstance(v, cfg.paramdef) else v

    def _setup(self, seed):
        I = self.ninst
        sizes = [int(np.prod(p.shape)) * I for p in self.tplugs]
        off = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        n = int(off[-1])
        self.P, self.dP, self.mP = (sm.zeros((n, 1), np.float32) for _ in range(3))
        self.drate, self.mrate = sm.zeros((n, 1), np.float32), sm.zeros((n, 1), np.float32)
        self.offsets, self.trnodes = off, []
        dll = _dll()
        dll.api_set_seed(int(seed))
        rate, mom = sm.asarray(self.rate), sm.asarray(self.momentum)
        for i, tp in enumerate(self.tplugs):
            shape = list(tp.shape)
            shape[tp.inst_axis] *= I
            sl = slice(int(off[i]), int(off[i + 1]))
            view = lambda vec: sarray(vec.tensor[sl].view(tuple(shape)), np.float32)
            flat = lambda vec: sarray(vec.tensor[sl], np.float32)
            tr = trainable(view(self.P), view(self.dP))
            connect(tr, tp)
            self.trnodes.append(tr)
            k = int(np.prod(tp.shape)) if tp.inst_axis == 0 else int(tp.shape[1])
            ones = sarray(torch.ones((sizes[i], 1), dtype=torch.float32, device=self.P.tensor.device), np.float32)
            dsm.madd_bcast(ones, rate, k, flat(self.drate))
            dsm.madd_bcast(ones, mom, k, flat(self.mrate))
            owner = tp.origin().node
            init = np.broadcast_to(np.asarray(self._draw(owner.init, np.random.default_rng(seed + 1 + i)), np.float32), (I,)).copy()
            noise = sm.empty((sizes[i], 1), np.float32)
            dll.db_randn(noise.data_ptr(), sizes[i])
            dsm.madd_bcast(noise, sm.asarray(init), k, flat(self.P))          # P = randn * init[instance]
            mu = getattr(owner, "init_mu", None)
            if mu is not None and np.any(np.asarray(mu) != 0):
                dsm.madd_bcast(ones, sm.asarray(np.broadcast_to(np.asarray(mu, np.float32), (I,)).copy()), k, flat(self.P))
        for t in self.trnodes:
            t.enforce_constraints()

    def param(self, name):
        """The parameter array feeding the trainable plug ``name`` of the cost graph."""
        for t, p in zip(self.trnodes, self.tplugs):
            if p.name == name:
                return t.P
        raise KeyError(name)

    def train_step(self, batch):
        """One step on ``batch`` = {plug name: device array} (X_seq, R_seq, F, Y, ...)."""
        flags.push("weight_decay_start", self.spec.weight_decay_start)
        flags.push("step", self.step)
        flags.push("train_mode", True)
        try:
            dsm.gradstep(self.P, self.dP, self.drate, self.mP, self.mrate,
                         grad=lambda: self.cost.bprop_trainable(self.trnodes, batch), nesterov=bool(self.spec.nesterov))
            for t in self.trnodes:
                t.enforce_constraints()
        finally:
            flags.pop("train_mode"); flags.pop("step"); flags.pop("weight_decay_start")
        self.step += 1

    def fit(self, batches, on_checkpoint=None):
        nb = len(batches)
        max_steps = int(min(self.spec.max_steps, self.spec.max_epochs * nb))
        cps = {int(max_steps * float(k) / self.spec.checkpoints) for k in range(1, int(self.spec.checkpoints) + 1)}
        for step in range(max_steps):
            self.train_step(batches[step % nb])
            if self.step in cps and on_checkpoint:
                on_checkpoint(self.step, self)
        return self

    def loss(self, batches):
        return self.cost.eval_loss(batches)

    def predict(self, batches):
        return self.cost.eval_model(batches)


def gradcheck(trainer, batch, nprobe=12, step=2e-3, rtol=5e-2, atol=1e-3, seed=0):
    """Compares the graph's gradient with central differences of the summed cost at a
    few parameters of every trainable node, in test mode (deepity/gradcheck.py:42-130;
    the reference perturbs by 1e-4 in float32 and accepts atol 1e-4; the step here is
    larger because the cost is a float32 mean, and small enough that few rectifiers
    switch within it).  Raises AssertionError listing the parameters that disagree."""
    rng = np.random.default_rng(seed)
    failures = []
    flags.push("gradcheck", True)
    try:
        trainer.cost.bprop_trainable(trainer.trnodes, batch)
        dP = trainer.dP.asnumpy().ravel().copy()

        def total_cost():
            trainer.cost._set(batch)
            c = trainer.cost.cost.fpval
            v = float(np.sum(c.asnumpy())) if isinstance(c, sarray) else float(np.sum(c))
            trainer.cost._unset(batch)
            return v
        for t, (lo, hi) in zip(trainer.trnodes, zip(trainer.offsets[:-1], trainer.offsets[1:])):
            for i in rng.choice(np.arange(lo, hi), size=min(nprobe, hi - lo), replace=False):
                x = float(trainer.P.tensor[i, 0])
                trainer.P.tensor[i, 0] = x - step; c0 = total_cost()
                trainer.P.tensor[i, 0] = x + step; c1 = total_cost()
                trainer.P.tensor[i, 0] = x
                num = (c1 - c0) / (2 * step)
                if not np.isclose(num, dP[i], rtol=rtol, atol=atol):
                    failures.append((t.Z.dsts[0].origin().path, int(i - lo), num, float(dP[i])))
    finally:
        flags.pop("gradcheck")
    if failures:
        raise AssertionError("gradient check failed:\n" + "\n".join("  %s[%d] numeric %.6g graph %.6g" % f for f in failures))
    return True
