"""Models and trainers written in the reference's config syntax.

A DeepBind model file (code/cfg/**/*.cfg) is a Python script that returns a list
of layer constructors -- ``motif_scan(...)``, ``bias()``, ``rectify()``,
``maxpool()``, ``dropout(rate=...)``, ``full(num_units=...)``, ``softmax()`` --
whose arguments may be hyper-parameter ranges (``loguniform(lo, hi)``,
``choice([...])``, ...); a trainer file returns ``sgd(...)``.  The reference
executes the script with every node type in scope, then rewrites the list into
a ``sequencenet`` graph of nodes and plugs
(code/libs/deepity/deepity/_io_/load.py:51-115,
code/libs/kangaroo/kangaroo/model.py:45-132).

Here the same script is executed against light-weight descriptors with the same
names and keyword arguments, and :func:`plan` recognises the layer sequence of
the DeepBind family as a whole,

    motif_scan bias rectify {max,avg,all}pool [dropout] full bias
                                              [rectify full bias] [softmax]

mapping ``motif_scan..pool`` onto the fused scan kernel and everything after the
pooling onto the fused dense head (:class:`deepbind_b200.model.DeepBindNet`).
:func:`instantiate` draws one hyper-parameter sample per model instance and
initialises the flat parameter vector as ``sgd._train_setup`` does
(code/libs/deepity/deepity/sgd.py:287-354).  The general node/plug graph engine
is not reproduced: a layer list outside this family raises NotImplementedError.
"""
import re

import numpy as np


# ------------------------------------------------------------ hyper-parameters
class paramdef(object):
    """A hyper-parameter range (code/libs/deepity/deepity/hpsearch.py:95-151);
    ``sample(rng, n)`` draws n values from a seeded numpy Generator."""

    def sample(self, rng, n):
        raise NotImplementedError


class choice(paramdef):
    def __init__(self, choices, name=None):
        assert len(choices) > 0
        self.choices, self.name = np.asarray(choices), name

    def sample(self, rng, n):
        return np.asarray([self.choices[rng.integers(0, len(self.choices))] for _ in range(n)])


class uniform(paramdef):
    def __init__(self, lo, hi, name=None):
        assert lo <= hi
        self.lo, self.hi, self.name = lo, hi, name

    def sample(self, rng, n):
        return np.asarray([float(rng.random() * (self.hi - self.lo) + self.lo) for _ in range(n)])


class loguniform(paramdef):
    """10 ** uniform(log10(lo), log10(hi))"""

    def __init__(self, lo, hi, name=None):
        assert lo <= hi
        self.lo, self.hi, self.name = lo, hi, name

    def sample(self, rng, n):
        lo, hi = np.log10(self.lo), np.log10(self.hi)
        return np.asarray([10 ** (rng.random() * (hi - lo) + lo) for _ in range(n)])


class powuniform(paramdef):
    """lo + (hi - lo) * uniform(0, 1) ** p, 0 < p <= 1"""

    def __init__(self, lo, hi, p, name=None):
        assert lo <= hi and 0 < p <= 1
        self.lo, self.hi, self.p, self.name = lo, hi, p, name

    def sample(self, rng, n):
        return np.asarray([float(rng.random() ** self.p * (self.hi - self.lo) + self.lo) for _ in range(n)])


class fixed(paramdef):
    """One given value per model (the best sample of an earlier search)."""

    def __init__(self, values, name=None):
        self.values, self.name = np.asarray(values), name

    def sample(self, rng, n):
        assert len(self.values) == n, "fixed() needs one value per model instance"
        return self.values


# ---------------------------------------------------------------------- layers
class layer(object):
    """Descriptor of one node of a model file; keeps its keyword arguments."""

    def __repr__(self):
        return "%s(%s)" % (type(self).__name__, ", ".join("%s=%r" % kv for kv in sorted(vars(self).items())))


class motif_scan(layer):
    """kangaroo/_ext/corr1ord.py:160-162.  ``motif_len`` defaults to ``num_motifs``
    there (the scripts then overwrite ``fsize``); :func:`instantiate` takes the
    final length as an argument for the same purpose."""

    def __init__(self, num_motifs, motif_len=None, weight_decay=0, init_scale=1e-3):
        self.num_motifs, self.motif_len = num_motifs, motif_len
        self.weight_decay, self.init_scale = weight_decay, init_scale


class bias(layer):
    def __init__(self, init=0.0, init_mu=0, negdecay=None, viz=True, start_training=0):      # elemwise.py:164
        self.init, self.init_mu, self.negdecay, self.start_training = init, init_mu, negdecay, start_training


class relu(layer):
    pass


class rectify(relu):
    pass


class maxpool(layer):
    pool = "max"


class avgpool(layer):
    pool = "avg"


class allpool(layer):
    pool = "all"


class dropout(layer):
    def __init__(self, rate=0.5, activerange=None):                                        # elemwise.py:122
        self.rate = rate


class full(layer):
    def __init__(self, num_units, weight_decay=None, init_scale=None, init_bias=None, ishape=None, oshape=None):   # full.py:48
        self.num_units = num_units
        self.weight_decay = weight_decay
        self.init_scale = init_scale if init_scale is not None else 0.001
        self.init_bias = init_bias if init_bias is not None else 0.0


class softmax(layer):
    """One column per model: the logistic function, trained with nll (softmax.py:50-61, loss.py:141-150)."""

    def __init__(self, ngroup=1):
        self.ngroup = ngroup


class logistic(layer):
    pass


class sgd(object):
    """Trainer descriptor with the reference's arguments and defaults (sgd.py:53-66);
    :class:`deepbind_b200.trainer.Trainer` runs it."""

    def __init__(self, rate=0.05, rate_decay=1.0, momentum=0.85, nesterov=True, batchsize=64, max_epochs=20,
                 max_steps=10000, viz_steps=10000, checkpoints=1, checkpoint_save=True, weight_decay_start=100,
                 lossfunc=None, gradcheck=False):
        self.rate, self.rate_decay, self.momentum, self.nesterov = rate, rate_decay, momentum, nesterov
        self.batchsize, self.max_epochs, self.max_steps = batchsize, max_epochs, max_steps
        self.checkpoints, self.weight_decay_start = checkpoints, weight_decay_start


_NAMESPACE = {c.__name__: c for c in (choice, uniform, loguniform, powuniform, fixed, motif_scan, bias, relu, rectify,
                                      maxpool, avgpool, allpool, dropout, full, softmax, logistic, sgd)}
_NAMESPACE["numpy"] = np


def loads(text, *args):
    """Executes config text; returns what it ``return``s (or the named variables)."""
    m = re.search(r"^return", text, re.MULTILINE)               # "return model" -> "__result = model" (load.py:104-107)
    if m:
        text = text[:m.start(0)] + "__result=" + text[m.end(0):]
    scope = {}
    exec(compile(text, "<cfg>", "exec"), dict(_NAMESPACE), scope)
    if "__result" in scope:
        return scope["__result"]
    if args:
        return tuple(scope[a] for a in args)
    return scope


def load(filename, *args):
    with open(filename) as f:
        return loads(f.read(), *args)


# --------------------------------------------------------------------- peephole
class ModelPlan(object):
    """The DeepBind family member a layer list describes."""

    def __init__(self, scan, pool, drop, fulls, loss):
        self.scan, self.pool, self.drop, self.fulls, self.loss = scan, pool, drop, fulls, loss
        self.hidden = fulls[0].num_units if len(fulls) == 2 else 0


def plan(layers):
    """Matches the layer list against
    motif_scan bias rectify pool [dropout] full bias [rectify full bias] [softmax|logistic]."""
    names = [("relu" if isinstance(l, relu) else "pool" if isinstance(l, (maxpool, avgpool, allpool)) else
              "sigm" if isinstance(l, (softmax, logistic)) else type(l).__name__) for l in layers]
    m = re.fullmatch(r"motif_scan bias relu pool (dropout )?full bias (relu full bias )?(sigm )?", " ".join(names) + " ")
    if not m:
        raise NotImplementedError("only the layer sequence motif_scan bias rectify {max,avg,all}pool [dropout] full bias "
                                  "[rectify full bias] [softmax] maps onto the fused kernels; got: " + " ".join(names))
    fulls = [l for l in layers if isinstance(l, full)]
    if fulls[-1].num_units != 1:
        raise NotImplementedError("the last full layer must have one unit per model")
    drops = [l for l in layers if isinstance(l, dropout)]
    return ModelPlan(layers[0], layers[3].pool, drops[0] if drops else None, fulls, "nll" if m.group(3) else "mse")


def select_instances(params, ids, ninst):
    """The parameter blocks of the instances ``ids`` cut out of blocks holding ``ninst``
    instances: filter and bias columns are instance-major (corr1ord.py:57-58), dense
    weights stack the instances on rows (full.py:57)."""
    out = {}
    for k, w in params.items():
        if k in ("W1", "W2"):
            out[k] = w.reshape(ninst, -1, w.shape[-1])[ids].reshape(-1, w.shape[-1])
        elif w.ndim == 2:
            out[k] = w.reshape(w.shape[0], ninst, -1)[:, ids].reshape(w.shape[0], -1)
        else:
            out[k] = w.reshape(ninst, -1)[ids].reshape(-1)
    return out


def _draw(value, rng, n, drawn, key):
    if isinstance(value, paramdef):
        drawn[key] = value.sample(rng, n)
        return np.asarray(drawn[key], np.float64)
    return np.full(n, 0.0 if value is None else value, np.float64)


def instantiate(layers, ninst=1, seed=0, motif_len=None, device=None, instances=None):
    """Builds ``ninst`` independent instances of the model in one DeepBindNet, one
    hyper-parameter draw per instance (as hypertrain trains its samples side by
    side, code/libs/deepity/deepity/hypertrain.py:560-580).

    Returns (net, drawn): ``drawn`` maps "<layer index>.<layer>.<argument>" to the [ninst]
    values drawn from a range.  Weights start as N(0, init_scale[instance]^2),
    biases at ``init_mu`` (sgd.py:331-352).  ``motif_len`` overrides the filter
    length the way the training scripts set ``fsize`` after loading.

    ``instances`` (a list of instance numbers < ninst): the net holds only those
    instances, with exactly the hyper-parameters and initial weights they have in the
    full net -- what a rank needs when the instances are dealt to several GPUs
    (hpsearch.py:316-330); ``drawn`` still lists all ``ninst`` draws."""
    from .model import DeepBindNet
    p = plan(layers)
    rng = np.random.default_rng(seed)
    drawn = {}
    I, F = ninst, p.scan.num_motifs
    m = motif_len or p.scan.motif_len or p.scan.num_motifs
    npool = F * (2 if p.pool == "all" else 1)
    idx = {id(l): i for i, l in enumerate(layers)}

    def draw(l, arg):
        return _draw(getattr(l, arg), rng, I, drawn, "%d.%s.%s" % (idx[id(l)], type(l).__name__, arg))

    scan_init, scan_decay = draw(p.scan, "init_scale"), draw(p.scan, "weight_decay")
    rate = draw(p.drop, "rate") if p.drop is not None else np.zeros(I)
    f_init = [draw(l, "init_scale") for l in p.fulls]
    f_decay = [draw(l, "weight_decay") for l in p.fulls]
    H = p.hidden
    params = {
        # filter columns are model-major: column = model * F + motif (corr1ord.py:57-58)
        "Wscan": (rng.standard_normal((4 * m, I, F)) * scan_init[None, :, None]).reshape(4 * m, I * F),
        "bscan": np.full(I * F, float(layers[1].init_mu)),
        # dense weights stack the models on rows (full.py:57)
        "W1": (rng.standard_normal((I, npool, H or 1)) * f_init[0][:, None, None]).reshape(I * npool, H or 1),
        "b1": np.full(I * (H or 1), float(p.fulls[0].init_bias)),
    }
    if H:
        params["W2"] = (rng.standard_normal((I, H, 1)) * f_init[1][:, None, None]).reshape(I * H, 1)
        params["b2"] = np.full(I, float(p.fulls[1].init_bias))
    params = {k: v.astype(np.float32) for k, v in params.items()}
    decay = {"Wscan": scan_decay, "W1": f_decay[0]}
    if H:
        decay["W2"] = f_decay[1]
    if instances is not None:
        ids = np.asarray(list(instances), np.int64)
        assert ids.size > 0 and ids.min() >= 0 and ids.max() < I, "instances must be numbers below ninst"
        params = select_instances(params, ids, I)
        decay = {k: v[ids] for k, v in decay.items()}
        scan_init, f_init, rate = scan_init[ids], [v[ids] for v in f_init], rate[ids]
        I = int(ids.size)
    net = DeepBindNet(params, I, p.pool, loss=p.loss, device=device)
    net.set_decay(decay)
    net.set_dropout(rate)
    net.hparams = {"dropout": rate, "decay": decay, "init": {"Wscan": scan_init, "W1": f_init[0]}}
    return net, drawn
