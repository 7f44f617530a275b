"""Minibatch trainer with the semantics of ``deepity.sgd``.

Nesterov momentum steps on the flat parameter vector of a
:class:`deepbind_b200.model.DeepBindNet` holding any number of independent
model instances, each with its own learning rate, momentum, dropout rate and
L1 weight decay (code/libs/deepity/deepity/sgd.py:87-163,287-354):

* minibatches are assembled once, up-front, and visited cyclically without
  reshuffling (sgd.py:92, ``asbatches(reshuffle=False)``);
* ``max_steps = min(max_steps, max_epochs * nbatch)`` and the checkpoint steps
  are ``max_steps * k / checkpoints`` (sgd.py:117-118);
* the L1 decay term is added from step ``weight_decay_start`` on
  (corr1ord.py:112-115, full.py:102-119);
* dropout draws one mask per step and model from the library's generator
  (``api_dropout_fp_tr``), or from uniform draws the caller supplies, which makes
  a run reproducible against the CPU restatement.

Batches, masks, forward, backward and update all run on the device; when every
minibatch has the same size the step is replayed from a CUDA graph.  With
``reverse_complement`` every sequence enters the minibatch on both strands, the
two rows share target and dropout mask, and only the stronger strand carries
loss and gradient (kangaroo/data.py:274-306, elemwise.py:140, loss.py:113-117).
"""
import numpy as np
import torch

from . import _lib, cfg, fused
from . import deepity_smat as dsm
from . import smat as sm


def _per_model(value, rng, I):
    if isinstance(value, cfg.paramdef):
        return np.asarray(value.sample(rng, I), np.float32)
    return np.broadcast_to(np.asarray(value, np.float32), (I,)).copy()


class Trainer(object):
    def __init__(self, net, spec=None, seed=0, ninst=None, instances=None, ministep=True):
        """``spec``: a :class:`deepbind_b200.cfg.sgd` (ranges are drawn once per model).
        ``ninst``/``instances``: the net holds the instances ``instances`` of a set of
        ``ninst`` (cfg.instantiate); rates are drawn for all and those kept, so that an
        instance trains the same on whichever GPU it lands."""
        self.net, self.spec = net, spec or cfg.sgd()
        rng = np.random.default_rng(seed)
        n = int(ninst) if ninst is not None else net.I
        self.rate_all = _per_model(self.spec.rate, rng, n)
        self.momentum_all = _per_model(self.spec.momentum, rng, n)
        ids = np.arange(n) if instances is None else np.asarray(list(instances), np.int64)
        assert len(ids) == net.I, "the net must hold exactly the listed instances"
        self.rate, self.momentum = self.rate_all[ids], self.momentum_all[ids]
        net.set_rates(self.rate, self.momentum)
        self.step = 0
        self.history = []                 # (step, mean training loss [I]) at every checkpoint
        self.reverse_complement = False   # set by fit()
        # small models train by the two-launch step (model.MiniStep) where it applies and its
        # per-sample gradient shares stay within a few megabytes; False forces the operator-fused step
        self.ministep = ministep

    # ------------------------------------------------------------------ data
    def make_batches(self, seqs, Y):
        """[(X, R, Y)] on the device, ``batchsize`` sequences each (the last one may be
        shorter).  Y [N] or [N, 1] is shared by all models; [N, I] gives one target
        column per model."""
        net, B = self.net, int(self.spec.batchsize)
        Y = np.asarray(Y, np.float32).reshape(len(seqs), -1)
        if Y.shape[1] == 1:
            Y = np.tile(Y, (1, net.I))
        assert Y.shape[1] == net.I, "targets must have one column, or one per model"
        batches = []
        rc = bool(self.reverse_complement)
        for lo in range(0, len(seqs), B):
            X, R = fused.build_batch(seqs[lo:lo + B], net.m - 1, rc, device=net.dev)
            Yb = np.repeat(Y[lo:lo + B], 2, axis=0) if rc else Y[lo:lo + B]       # both strands share the target
            batches.append((X, R, torch.from_numpy(np.ascontiguousarray(Yb)).to(net.dev)))
        return batches

    def _mask(self, nrow, draws):
        """Keep-mask [nrow, npool*I] of one step, or None without dropout."""
        net = self.net
        if net.dropout_rate is None:
            return None
        ones = sm.sarray(torch.ones((nrow, self._mask_cols()), dtype=torch.float32, device=net.dev), np.float32)
        U = None if draws is None else sm.sarray(draws, np.float32)
        _, M = dsm.dropout_fp_train(ones, sm.asarray(net.dropout_rate), bool(self.reverse_complement), U)
        return M.tensor

    # ------------------------------------------------------------------- loop
    def fit(self, seqs, Y, uniform_draws=None, on_checkpoint=None, use_graph=True, reverse_complement=False):
        """Trains for the trainer's step budget; returns the loss [I] of the last step.
        ``reverse_complement``: train on both strands of every sequence.

        ``uniform_draws(step, shape)`` (optional) returns the U(0,1) draws of that
        step's dropout mask as a CUDA f32 tensor; ``on_checkpoint(step, trainer)`` is
        called at every checkpoint after the mean training loss was recorded."""
        net, spec = self.net, self.spec
        self.reverse_complement = bool(reverse_complement)
        net.strand_pairs = self.reverse_complement
        batches = self.make_batches(seqs, Y)
        nb = len(batches)
        max_steps = int(min(spec.max_steps, spec.max_epochs * nb))
        checkpoints = {int(max_steps * float(k) / spec.checkpoints) for k in range(1, int(spec.checkpoints) + 1)}
        # Minibatches shaped like the first one (all of them, or all but a shorter last one) run
        # as a captured step; a last minibatch of another shape runs call by call.
        nfull = 0
        while nfull < nb and batches[nfull][0].numel() == batches[0][0].numel() and batches[nfull][1].shape == batches[0][1].shape:
            nfull += 1
        graphs = {}
        static = feed = mstep = None
        if use_graph and nfull >= max(1, nb - 1) and uniform_draws is None:
            X0, R0, Y0 = batches[0]
            static = (X0.clone(), R0.clone(), Y0.clone(), self._mask(R0.shape[0], None))
            # the captured step fetches the next of the stacked full minibatches by itself
            feed = fused.MinibatchFeed([(torch.stack([b[0] for b in batches[:nfull]]), static[0]),
                                        (torch.stack([b[1] for b in batches[:nfull]]), static[1]),
                                        (torch.stack([b[2] for b in batches[:nfull]]), static[2])])
            if static[3] is not None:
                # the step's dropout mask is drawn by a kernel of the graph (draw counter on the device)
                rate_dev = torch.from_numpy(np.ascontiguousarray(net.dropout_rate, np.float32)).to(net.dev)
                mask_counters = torch.zeros(2, dtype=torch.int32, device=net.dev)
                sM0 = static[3]

                def draw_mask():
                    sm.bind_stream()
                    _lib.load().db_dropout_mask(sM0.data_ptr(), sM0.shape[0], sM0.shape[1], rate_dev.data_ptr(), net.I,
                                                int(self.reverse_complement), mask_counters.data_ptr())
            sMask = static[3]
            if self.ministep:
                Rst = feed.pairs[1][0]
                max_rows = int((Rst[..., 1] - Rst[..., 0]).max())
                cand = net.ministep(feed.pairs[0][0], feed.pairs[1][0], feed.pairs[2][0], sMask, max_rows=max_rows)
                if cand is not None and cand.scratch_bytes <= (8 << 20):
                    mstep = cand
        loss = None
        ms_count = 0     # what the two-launch step's device-side counter holds
        K = 8            # steps per replay where a run of K steps allows it: a replay costs the host more than a small step
        cps = sorted(checkpoints)
        step = 0
        while step < max_steps:
            X, R, Yb = batches[step % nb]
            net.decay_on = step >= spec.weight_decay_start
            ran = 1
            if static is not None and step % nb < nfull:
                sX, sR, sY, sM = static
                # K steps in one replay if none of them is the short minibatch, switches the decay on,
                # or passes a checkpoint before the run's last step
                nextcp = next((c for c in cps if c > step), max_steps)
                many = (step % nb) + K <= nfull and step + K <= min(max_steps, nextcp) and \
                    (step >= spec.weight_decay_start or step + K <= spec.weight_decay_start)
                key = (bool(net.decay_on), K if many else 1)
                if key not in graphs and mstep is not None:
                    graphs[key] = (mstep.capture(steps=key[1], prologue=draw_mask if sM is not None else None), mstep.loss)
                if mstep is not None:                   # the step counter of the resident dataset, as run so far
                    want = (step // nb) * nfull + min(step % nb, nfull)
                    if want != ms_count:
                        mstep.counters[0] = want
                    ms_count = want + key[1]
                if key not in graphs:
                    # the capture's warm-up steps are real steps: put the state back afterwards
                    P0, mP0 = net.P.clone(), net.mP.clone()
                    graphs[key] = net.capture_train_step(sX, sR, sY, sM, warmup=1 if graphs else 3, feed=feed,
                                                         prologue=draw_mask if sM is not None else None, steps=key[1])
                    net.P.copy_(P0); net.mP.copy_(mP0)
                    feed.counters[0] = (step // nb) * nfull + min(step % nb, nfull)     # captured steps run so far
                graphs[key][0].replay()
                loss = graphs[key][1]
                ran = key[1]
            else:
                draws = uniform_draws(step, (R.shape[0], self._mask_cols())) if uniform_draws else None
                loss = net.train_step(X, R, Yb, self._mask(R.shape[0], draws))
            step += ran
            self.step = step
            if self.step in checkpoints:
                self.history.append((self.step, self.evaluate(batches[:100])))
                if on_checkpoint:
                    on_checkpoint(self.step, self)
        net.decay_on = False
        return loss

    def _mask_cols(self):
        net = self.net
        return (net.nf // net.I) * (2 if net.pool == "all" else 1) * net.I

    def evaluate(self, batches):
        """Mean loss [I] over the batches in test mode (dropout as scaling), as the
        progress report of sgd.py:165-188 computes it."""
        net = self.net
        dll = _lib.load()
        total = torch.zeros(net.I, dtype=torch.float32, device=net.dev)
        for X, R, Yb in batches:
            out = net.score(X, R).contiguous()
            lossv = torch.empty(net.I, dtype=torch.float32, device=net.dev)
            if net.loss == "nll":
                dll.db_logistic(out.data_ptr(), out.data_ptr(), out.numel())
            zmask = None
            if self.reverse_complement:     # only the stronger strand of a pair counts; the mean is over all rows
                zmask = torch.zeros(out.shape, dtype=torch.bool, device=net.dev)
                dsm.calc_Zmask(sm.sarray(out, np.float32), sm.sarray(zmask, np.bool_))
            dll.db_loss(1 if net.loss == "nll" else 0, out.data_ptr(), Yb.data_ptr(), None,
                        zmask.data_ptr() if zmask is not None else None, out.shape[0], net.I, lossv.data_ptr(), None)
            total += lossv
        return (total / max(1, len(batches))).cpu().numpy()
