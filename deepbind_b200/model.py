"""DeepBind networks assembled from the hot-path operators.

``DeepBindNet`` holds ``nmodel`` independent models (the reference's "instance"
axis, code/libs/deepity/deepity/hypertrain.py:576) in one flat parameter vector
``P`` with its gradient ``dP``, momentum ``mP`` and per-element rates, as
``sgd._train_setup`` lays them out (code/libs/deepity/deepity/sgd.py:287-354),
and runs

    scan -> bias -> rectify -> pool -> [dropout] -> full -> bias
         [-> rectify -> full -> bias] [-> logistic] -> loss

forward, backward and the Nesterov update entirely through libdeepbind_b200.so.
It is the composite the benchmark and parity tests drive, mapped as a whole onto
the fused kernels; the reference's node/plug graph engine, which runs the same
layers operator by operator, is ``deepbind_b200.graph``.
"""
import ctypes

import numpy as np
import torch

from . import _lib, fused
from . import deepity_smat as dsm
from .smat import sarray, bind_stream
from .smat import asarray as sm_asarray

ORDER = ("Wscan", "bscan", "W1", "b1", "W2", "b2")


def _as_f32(t):
    return sarray(t, np.float32)


class DeepBindNet(object):
    def __init__(self, params, nmodel, pool="max", loss="nll", device=None, fused_head=True):
        self.dev = device or torch.device("cuda", torch.cuda.current_device())
        self.fused_head = fused_head      # False: run the head operator by operator, as the reference's graph does
        self.I = int(nmodel)
        self.pool = pool
        self.loss = loss
        self.m = params["Wscan"].shape[0] // 4
        self.nf = params["Wscan"].shape[1]
        self.hidden = params["W1"].shape[1] if "W2" in params else 0
        self.names = [k for k in ORDER if k in params]
        self.shapes = {k: tuple(np.atleast_1d(params[k]).shape) for k in self.names}
        sizes = [int(np.prod(self.shapes[k])) for k in self.names]
        self.offsets = np.concatenate([[0], np.cumsum(sizes)])
        n = int(self.offsets[-1])
        host = np.concatenate([np.asarray(params[k], np.float32).ravel() for k in self.names])
        self.P = torch.from_numpy(host).to(self.dev)
        self.dP = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.mP = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.drate = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self.mrate = torch.zeros(n, dtype=torch.float32, device=self.dev)
        self._s = {k: _as_f32(getattr(self, k)) for k in ("P", "dP", "mP", "drate", "mrate")}
        self.decay = None                 # per-element L1 decay (set_decay); applied while decay_on
        self.decay_on = False
        self.dropout_rate = None          # per-model dropout rate of the pooled features (set_dropout)
        self.strand_pairs = False         # training rows are forward / reverse-complement pairs (grads masks the weaker strand)

    # ------------------------------------------------------------- parameters
    def _spread(self, vec, name, values, k=None):
        """vec[block of `name`] += values[model], model-wise, with madd_bcast as
        sgd.py:322-329 does (instance axis 0 for dense weights, 1 elsewhere)."""
        shp = self.shapes[name]
        inst_axis0 = name in ("W1", "W2")
        if k is None:
            k = int(np.prod(shp)) // self.I if inst_axis0 else (shp[-1] // self.I)
        i = self.names.index(name)
        seg = vec[int(self.offsets[i]):int(self.offsets[i + 1])]
        dsm.madd_bcast(_as_f32(torch.ones_like(seg)), np.array(values, np.float32), k, _as_f32(seg))

    def set_decay(self, decay):
        """L1 weight decay per model: ``decay`` maps a weight block ("Wscan", "W1",
        "W2") to a scalar or [I] array; biases are not decayed (corr1ord.py:112-126,
        full.py:102-119).  The term is added by grads() while ``decay_on`` is True
        (the trainer switches it on at ``weight_decay_start``).  For the filter bank
        the reference spreads the per-model values with k = rows / ninst
        (corr1ord.py:126), which with several models does not follow the
        model-major column layout; the same k is used here so that results agree."""
        self.decay = torch.zeros_like(self.P)
        for name, val in decay.items():
            if name in self.names and val is not None:
                k = max(1, self.shapes[name][0] // self.I) if name == "Wscan" else None
                self._spread(self.decay, name, np.broadcast_to(np.asarray(val, np.float32), (self.I,)), k)

    def set_dropout(self, rate):
        """Dropout rate of the pooled features, scalar or one per model.  Training
        masks are drawn by the trainer; scoring multiplies the pooled features by
        1 - rate instead (elemwise.py:128-150: no rescaling while training)."""
        rate = np.broadcast_to(np.asarray(rate, np.float32), (self.I,)).copy()
        self.dropout_rate = rate if np.any(rate > 0) else None
    def view(self, name, of="P"):
        i = self.names.index(name)
        t = getattr(self, of)[int(self.offsets[i]):int(self.offsets[i + 1])]
        shp = self.shapes[name]
        return t.view(shp) if len(shp) == 2 else t.view(1, -1)

    def set_rates(self, rate, momentum):
        """Per-model learning / momentum rates broadcast over each parameter block
        with madd_bcast, as sgd.py:322-329 does (instance axis 0 for dense
        weights, 1 elsewhere)."""
        rate = np.broadcast_to(np.asarray(rate, np.float32), (self.I,)).copy()
        momentum = np.broadcast_to(np.asarray(momentum, np.float32), (self.I,)).copy()
        self.drate.zero_(); self.mrate.zero_()
        for name in self.names:
            shp = self.shapes[name]
            inst_axis0 = name in ("W1", "W2")
            k = int(np.prod(shp)) // self.I if inst_axis0 else (shp[-1] // self.I)
            for vec, val in ((self.drate, rate), (self.mrate, momentum)):
                i = self.names.index(name)
                seg = vec[int(self.offsets[i]):int(self.offsets[i + 1])]
                ones = torch.ones_like(seg)
                dsm.madd_bcast(_as_f32(ones), val, k, _as_f32(seg))

    # ---------------------------------------------------------------- forward
    def _head(self, pooled):
        """Dense layers on pooled features [B, npool*I] -> pre-activation output [B, I]."""
        I = self.I
        dll = _lib.load()
        W1, b1 = self.view("W1"), self.view("b1")
        h1 = dsm.blockwise_dot(_as_f32(pooled), _as_f32(W1), I).tensor
        dll.db_bias_add(h1.data_ptr(), h1.data_ptr(), b1.data_ptr(), h1.shape[0], h1.shape[1])
        if not self.hidden:
            return h1, None, None
        a1 = torch.empty_like(h1)
        dll.db_relu(a1.data_ptr(), h1.data_ptr(), h1.numel())
        W2, b2 = self.view("W2"), self.view("b2")
        out = dsm.blockwise_dot(_as_f32(a1), _as_f32(W2), I).tensor
        dll.db_bias_add(out.data_ptr(), out.data_ptr(), b2.data_ptr(), out.shape[0], out.shape[1])
        return out, h1, a1

    def _test_dropout(self, pooled):
        """Scoring with a dropout layer: Z = X * (1 - rate[model]) (dropout.cu:64-75)."""
        if self.dropout_rate is None:
            return pooled
        return dsm.dropout_fp_test(_as_f32(pooled), sm_asarray(self.dropout_rate)).tensor

    def score(self, X, R, strand_max=False):
        """Scores [nseq, I] (no output non-linearity).  With strand_max, rows are
        fwd/rc pairs and the larger score of each pair is kept, forward on ties
        (code/libs/kangaroo/kangaroo/predict.py:145-164)."""
        bind_stream()
        pooled, _, _ = fused.scanpool(self.view("Wscan"), self.view("bscan").view(-1), X, R, self.pool, relu=True)
        out, _, _ = self._head(self._test_dropout(pooled))
        if strand_max:
            both = out.contiguous()
            out = torch.empty((both.shape[0] // 2, self.I), dtype=torch.float32, device=self.dev)
            _lib.load().db_strand_max(out.data_ptr(), both.data_ptr(), out.shape[0], self.I)
        return out

    def input_gradients(self, X, R, strand_max=False):
        """Gradient maps of kangaroo.predict (code/libs/kangaroo/kangaroo/predict.py:168-265,
        deepity/node.py:317-338): the output Z (after the logistic for an nll model) is fed
        back as dZ = Z - 0 with no minibatch mean, through the dense layers in test mode,
        pooling, rectifier and scan, down to dX [npos, 4].  With strand_max only the
        stronger row of each forward / reverse-complement pair feeds back.  Runs the
        drop-in operators one by one (the activation [npos, nf] is materialised), as the
        reference does.  Returns (Z [nrow, I], dX)."""
        from . import kangaroo_smat as ks
        bind_stream()
        dll = _lib.load()
        I = self.I
        W, b = self.view("Wscan").contiguous(), self.view("bscan").view(-1)
        sX, sR = sarray(X.view(-1, 1), np.uint8), sarray(R.view(torch.int32), np.uint32)
        act = torch.zeros((X.numel(), self.nf), dtype=torch.float32, device=self.dev)
        ks.corr1ord(_as_f32(W), sX, _as_f32(act), 4)
        dll.db_bias_add(act.data_ptr(), act.data_ptr(), b.data_ptr(), act.shape[0], act.shape[1])
        dll.db_relu(act.data_ptr(), act.data_ptr(), act.numel())
        pooled, amax = ks.poolrgn(_as_f32(act), sR, self.pool, want_argmax=self.pool in ("max", "all"))
        out, h1, a1 = self._head(self._test_dropout(pooled.tensor))
        Z = out.clone()
        if self.loss == "nll":
            dll.db_logistic(Z.data_ptr(), out.data_ptr(), out.numel())
        dZ = Z.clone()
        if strand_max:
            z = Z.view(-1, 2, I)
            fwd = z[:, 0] >= z[:, 1]
            dZ = torch.where(torch.stack([fwd, ~fwd], 1).reshape(-1, I), dZ, torch.zeros_like(dZ))
        if self.hidden:
            da1 = dsm.blockwise_dot_nt(_as_f32(dZ.contiguous()), _as_f32(self.view("W2")), I).tensor
            dh = torch.empty_like(da1)
            dll.db_relu_bprop(dh.data_ptr(), da1.data_ptr(), a1.data_ptr(), dh.numel())
        else:
            dh = dZ.contiguous()
        dpd = dsm.blockwise_dot_nt(_as_f32(dh), _as_f32(self.view("W1")), I)
        if self.dropout_rate is not None:
            dpd = dsm.dropout_bp_te(dpd, sm_asarray(self.dropout_rate))
        dact = torch.zeros_like(act)
        ks.poolrgn_bprop(_as_f32(dact), sR, dpd, amax, self.pool)
        dll.db_relu_bprop(dact.data_ptr(), dact.data_ptr(), act.data_ptr(), dact.numel())
        dX = torch.zeros((X.numel(), 4), dtype=torch.float32, device=self.dev)
        ks.corr1ord_bprop_X(_as_f32(dX), _as_f32(W), _as_f32(dact), 4)
        return Z, dX

    # --------------------------------------------------------------- backward
    def grads(self, X, R, Y, dropmask=None):
        """Fills dP with the gradient of the mean loss at P; returns loss [I].
        Y is [B, I] f32; dropmask (optional, bool [B, npool*I]) is the dropout
        keep-mask applied to the pooled features.  While ``decay_on`` is set, the L1
        weight-decay term decay * sign(W) is added (set_decay)."""
        lossv = self._grads(X, R, Y, dropmask)
        if self.decay_on and self.decay is not None:
            _lib.load().db_l1_decay(self.dP.data_ptr(), self.P.data_ptr(), self.decay.data_ptr(), self.P.numel())
        return lossv

    def _grads(self, X, R, Y, dropmask=None):
        bind_stream()
        I = self.I
        dll = _lib.load()
        pooled, amax, actmask = fused.scanpool(self.view("Wscan"), self.view("bscan").view(-1), X, R, self.pool,
                                               relu=True, want_argmax=True, want_actmask=True)
        B = pooled.shape[0]
        npool = pooled.shape[1] // I
        if self.fused_head and B <= dll.db_head_max_batch(npool, self.hidden):
            # dense head, loss and their backward pass in one launch; gradients land in dP
            lossv = torch.empty(I, dtype=torch.float32, device=self.dev)
            dpd = torch.empty_like(pooled)
            has2 = bool(self.hidden)
            dll.db_head_train(I, npool, self.hidden, 1 if self.loss == "nll" else 0, int(self.strand_pairs), B, pooled.data_ptr(),
                              dropmask.data_ptr() if dropmask is not None else None, Y.data_ptr(),
                              self.view("W1").data_ptr(), self.view("b1").data_ptr(),
                              self.view("W2").data_ptr() if has2 else None, self.view("b2").data_ptr() if has2 else None,
                              lossv.data_ptr(), dpd.data_ptr(), self.view("W1", "dP").data_ptr(),
                              self.view("b1", "dP").data_ptr(),
                              self.view("W2", "dP").data_ptr() if has2 else None,
                              self.view("b2", "dP").data_ptr() if has2 else None)
            dW, db = fused.scanpool_bprop(self.m, self.nf, X, R, self.pool, dpd, amax, actmask,
                                          dW_out=self.view("Wscan", "dP"), db_out=self.view("bscan", "dP").view(-1))
            return lossv
        if dropmask is not None:
            pd = pooled.clone()
            dsm.maskout(sarray(dropmask, np.bool_), _as_f32(pd))
        else:
            pd = pooled
        out, h1, a1 = self._head(pd)
        B = out.shape[0]
        lossv = torch.empty(I, dtype=torch.float32, device=self.dev)
        dout = torch.empty_like(out)
        z = out
        if self.loss == "nll":
            z = torch.empty_like(out)
            dll.db_logistic(z.data_ptr(), out.data_ptr(), out.numel())
        zmask = None
        if self.strand_pairs:               # the stronger strand of each row pair carries loss and gradient (loss.py:113-117)
            zmask = torch.zeros(out.shape, dtype=torch.bool, device=self.dev)
            dsm.calc_Zmask(_as_f32(z), sarray(zmask, np.bool_))
        dll.db_loss(1 if self.loss == "nll" else 0, z.data_ptr(), Y.data_ptr(), None,
                    zmask.data_ptr() if zmask is not None else None, B, I, lossv.data_ptr(), dout.data_ptr())
        if self.hidden:
            W2 = self.view("W2")
            dll.db_colsum(self.view("b2", "dP").data_ptr(), dout.data_ptr(), B, I)
            dW2 = dsm.blockwise_dot_tn(_as_f32(a1), _as_f32(dout), I, _as_f32(W2)).tensor
            self.view("W2", "dP").copy_(dW2)
            da1 = dsm.blockwise_dot_nt(_as_f32(dout), _as_f32(W2), I).tensor
            dh1 = torch.empty_like(da1)
            dll.db_relu_bprop(dh1.data_ptr(), da1.data_ptr(), a1.data_ptr(), a1.numel())
        else:
            dh1 = dout
        W1 = self.view("W1")
        dll.db_colsum(self.view("b1", "dP").data_ptr(), dh1.data_ptr(), B, dh1.shape[1])
        dW1 = dsm.blockwise_dot_tn(_as_f32(pd), _as_f32(dh1), I, _as_f32(W1)).tensor
        self.view("W1", "dP").copy_(dW1)
        dpd = dsm.blockwise_dot_nt(_as_f32(dh1), _as_f32(W1), I).tensor
        if dropmask is not None:
            dsm.maskout(sarray(dropmask, np.bool_), _as_f32(dpd))
        dW, db = fused.scanpool_bprop(self.m, self.nf, X, R, self.pool, dpd, amax, actmask)
        self.view("Wscan", "dP").copy_(dW)
        self.view("bscan", "dP").view(-1).copy_(db)
        return lossv

    def train_step(self, X, R, Y, dropmask=None):
        """One Nesterov step (deepity_smat.py:98-109): look-ahead, gradient, update."""
        out = {}
        dsm.gradstep(self._s["P"], self._s["dP"], self._s["drate"], self._s["mP"], self._s["mrate"],
                     grad=lambda: out.setdefault("loss", self.grads(X, R, Y, dropmask)), nesterov=True)
        return out["loss"]

    def ministep(self, X, R, Y, dropmask=None, order=None, max_rows=None):
        """The two-launch training step over a minibatch or a device-resident dataset
        (see :class:`MiniStep`); None when the model or the shapes are outside it."""
        ms = MiniStep(self, X, R, Y, dropmask, order, max_rows)
        return ms if ms.supported else None

    # ------------------------------------------------------ tensor-core scoring
    def prepare_tc(self, precision="f16x2"):
        """Prepares the filter bank for the tcgen05 scan (redo after a weight change)."""
        self._tcw = fused.TCWeights(self.view("Wscan").contiguous(), self.view("bscan").view(-1), precision)
        return self._tcw

    def score_tc(self, X, R, strand_max=False, check=True, out=None, status=None):
        """Scores [nseq, I] through the tensor-core scan.  With a linear head the
        head is applied inside the kernel and no pooled features reach HBM."""
        bind_stream()
        tcw = getattr(self, "_tcw", None) or self.prepare_tc()
        if not self.hidden and self.nf == 16 * self.I and self.dropout_rate is None:
            _, out = fused.scanpool_tc(tcw, X, R, self.pool, headW=self.view("W1").reshape(-1),
                                       headB=self.view("b1").view(-1), check=check, scores_out=out, status=status)
        else:
            pooled, _ = fused.scanpool_tc(tcw, X, R, self.pool, check=check, status=status)
            res, _, _ = self._head(self._test_dropout(pooled))
            if out is not None:                 # the caller's buffer is honoured on every branch
                out.copy_(res.view(out.shape))
            else:
                out = res
        if strand_max:
            both = out.contiguous()
            out = torch.empty((both.shape[0] // 2, self.I), dtype=torch.float32, device=self.dev)
            _lib.load().db_strand_max(out.data_ptr(), both.data_ptr(), out.shape[0], self.I)
        return out

    def score_chunked(self, X, R, out, chunk=16384):
        """Scores every region of a device-resident batch into ``out`` [nseq, I],
        ``chunk`` sequences at a time so that the pooled features (npool*I floats
        per sequence) never need more than one chunk of HBM."""
        nseq = R.shape[0]
        for s in range(0, nseq, chunk):
            e = min(nseq, s + chunk)
            out[s:e].copy_(self.score(X, R[s:e]))
        return out

    def predict_host(self, X_host, R_host, out_host, chunk=16384, dev_bufs=None, tc=False, npiece=16, on_piece=None, before_piece=None,
                     wait=True):
        """The call a user makes for scoring: ordinal batch in (pinned) host
        memory -> scores in (pinned) host memory.  Mirrors what
        kangaroo.predict does per batch (code/libs/kangaroo/kangaroo/predict.py:168-176):
        upload X and R, run the model, read the scores back.  On the pipelined
        tensor-core path the batch is cut into ``npiece`` pieces of regions
        (``shard.shard_range(nseq, c, npiece)``) and ``on_piece(lo, hi)``, if given, is
        called right after piece [lo, hi) was enqueued on the current stream (a caller
        with several GPUs starts that piece's all-gather there); ``before_piece(lo, hi)``
        is called just before the piece's scan is enqueued.

        ``wait=False`` (pipelined path only) returns as soon as everything is enqueued:
        a caller streaming batch after batch through the same device buffers calls
        again at once, and the next batch's uploads and scans run while this batch's
        last scores are still on their way to the host (piece c of the next call waits
        only for piece c of this one: its scan for the upload, its read-back for the
        scan); :meth:`predict_host_wait` synchronises and raises if any scan since the
        last wait failed (a failed scan makes the later ones return at once)."""
        if dev_bufs is None:
            dev_bufs = (torch.empty(X_host.shape, dtype=torch.uint8, device=self.dev),
                        torch.empty(R_host.shape, dtype=torch.int32, device=self.dev),
                        torch.empty(out_host.shape, dtype=torch.float32, device=self.dev))
        X, R, out = dev_bufs
        cur = torch.cuda.current_stream()
        if tc:
            if not hasattr(self, "_status"):
                self._status = torch.zeros(1, dtype=torch.int32, device=self.dev)
            if getattr(self, "_pipe", None) is None:
                self._status.zero_()            # a failure of an earlier, finished call must not outlive it
        if tc and self.hidden == 0 and self.nf == 16 * self.I and self.dropout_rate is None and R.shape[0] >= 8 * 4096:
            # Both transfers are pipelined with the scan, piece by piece: the bases of the next
            # piece go up on one side stream and the scores of the last piece come back on another
            # while the current piece is scanned; the 4*I bytes per sequence of the read-back
            # otherwise add their full PCIe time to the step.
            if not hasattr(self, "_copy_stream"):
                self._copy_stream = torch.cuda.Stream(device=self.dev)
                self._up_stream = torch.cuda.Stream(device=self.dev)
            R.copy_(R_host, non_blocking=True)
            from .shard import shard_range
            nseq, npos = R.shape[0], X.numel()
            npiece = max(1, min(int(npiece), nseq))
            cuts = [shard_range(nseq, c, npiece)[0] for c in range(npiece)] + [nseq]
            first = [int(R_host[lo, 0]) for lo in cuts[:-1]] + [npos]          # regions ascend (the batch layout)
            # a call still in flight on the same buffers and cuts: piece by piece dependencies; anything else: all of it first
            key = (X.data_ptr(), out.data_ptr(), tuple(cuts))
            prev = getattr(self, "_pipe", None)
            if prev is not None and prev["key"] != key:
                self.predict_host_wait()
                prev = None
            if prev is None:
                self._up_stream.wait_stream(cur)
            ups, dones, reads = [], [], []
            with torch.cuda.stream(self._up_stream):
                for c in range(npiece):
                    if prev is not None:            # the rows this upload overwrites were read by scans c and c+1 of the call before
                        self._up_stream.wait_event(prev["done"][min(c + 1, npiece - 1)])
                    a0, a1 = first[c], min(npos, first[c + 1] + self.m - 1)    # the piece's rows and the taps' reach past them
                    X[a0:a1].copy_(X_host[a0:a1], non_blocking=True)
                    ev = torch.cuda.Event(); ev.record(self._up_stream); ups.append(ev)
            for c in range(npiece):
                lo, hi = cuts[c], cuts[c + 1]
                cur.wait_event(ups[c])
                if prev is not None:
                    cur.wait_event(prev["read"][c])  # the scores this scan overwrites have reached the host
                if before_piece is not None:
                    before_piece(lo, hi)
                self.score_tc(X, R[lo:hi], check=False, out=out[lo:hi], status=self._status)
                if on_piece is not None:
                    on_piece(lo, hi)
                done = torch.cuda.Event()
                done.record(cur)
                dones.append(done)
                self._copy_stream.wait_event(done)
                with torch.cuda.stream(self._copy_stream):
                    out_host[lo:hi].copy_(out[lo:hi], non_blocking=True)
                    rd = torch.cuda.Event(); rd.record(self._copy_stream); reads.append(rd)
            self._pipe = {"key": key, "done": dones, "read": reads}
            if wait:
                self.predict_host_wait()
            return out_host
        X.copy_(X_host, non_blocking=True)
        R.copy_(R_host, non_blocking=True)
        if tc:
            if before_piece is not None:
                before_piece(0, R.shape[0])
            self.score_tc(X, R, check=False, out=out, status=self._status)
        else:
            self.score_chunked(X, R, out, chunk)
        out_host.copy_(out, non_blocking=True)
        cur.synchronize()
        if tc:
            self._check_tc_status()
        return out_host

    def predict_host_wait(self):
        """Waits for every :meth:`predict_host` call enqueued with ``wait=False`` and raises if
        a scan among them failed."""
        if getattr(self, "_pipe", None) is None:
            return
        self._copy_stream.synchronize()
        torch.cuda.current_stream().synchronize()
        self._pipe = None
        self._check_tc_status()

    def _check_tc_status(self):
        """Raises if a tensor-core scan of the call just synchronised gave up (1 = a
        bounded wait ran out, 3 = regions not in ascending order)."""
        st = int(self._status.item())
        if st != 0:
            self._status.zero_()
            raise _lib.SmatException("scanpool_tc(...) raised an exception\nRuntimeError: tensor-core scan failed (status %d)" % st)

    def capture_train_step(self, X, R, Y, dropmask=None, warmup=3, feed=None, prologue=None, steps=1):
        """Captures one Nesterov step on the static buffers X, R, Y, dropmask into a
        CUDA graph and returns (graph, loss): refill the buffers in place (same
        shapes) and call ``graph.replay()`` for every further step.  A minibatch
        step is some twenty small kernels; replaying them as one graph removes the
        per-launch host cost that otherwise dominates (the reference pays it on
        every step, 40-60 ctypes calls each).  The warm-up steps run first on a
        side stream so that the library's scratch buffer has its final size: no
        allocation may happen while a stream is being captured.  With ``feed`` (a
        fused.MinibatchFeed whose step buffers are X, Y, dropmask) the graph first
        fetches the next minibatch of the device-resident dataset, so replaying it
        walks the dataset with no host work between steps; the feed's step counter is
        back at zero when this returns.  ``prologue`` (a callable launching further
        kernels, e.g. the draw of the step's dropout mask into ``dropmask``) runs inside
        the graph between the fetch and the step.  ``steps`` > 1 (with a feed) captures that
        many consecutive steps into the one graph: a replay of a small model's step costs
        the host more than the step takes on the GPU, and several steps per replay bring
        the loop back to the GPU's pace; ``loss`` is then that of the last step."""
        assert steps == 1 or feed is not None, "several steps per graph need a feed that advances by itself"
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(warmup):
                if feed is not None:
                    feed.fetch()
                if prologue is not None:
                    prologue()
                self.train_step(X, R, Y, dropmask)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        if feed is not None:
            feed.counters.zero_()
            torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(steps):
                if feed is not None:
                    feed.fetch()
                if prologue is not None:
                    prologue()
                loss = self.train_step(X, R, Y, dropmask)
        return graph, loss

    def capture_score(self, X, R, strand_max=False, warmup=3):
        """Captures ``score`` on the static buffers X, R into a CUDA graph and returns
        (graph, scores): refill X and R in place (same shapes) and ``graph.replay()``.
        For small batches (a 4096-probe PBM chunk is under 100 M adds) the scan is a
        few microseconds and the host cost of the separate launches dominates."""
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.score(X, R, strand_max)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.score(X, R, strand_max)
        return graph, out

    def params_numpy(self, of="P"):
        return {k: self.view(k, of).detach().cpu().numpy().reshape(self.shapes[k]) for k in self.names}


POOL_CODE = {"max": 0, "avg": 1, "sum": 2, "all": 3}


class MiniStep(object):
    """One Nesterov step of a small model as two launches (``db_ministep``): a CTA per
    (sample or strand pair, model) runs the whole layer chain forward and backward for its
    sample in shared memory, and an update kernel adds the samples' gradient shares, applies
    L1 decay and the update of deepity_smat/gradstep.cu:41-72 and writes the next step's
    look-ahead parameters -- against seven launches of the operator-fused path
    (:meth:`DeepBindNet.train_step`), whose latencies are what a small step consists of.

    ``X`` [npos] u8, ``R`` [B, 2], ``Y`` [B, I], ``dropmask`` [B, npool*I] bool: one
    minibatch; or each with a leading axis [nbatch, ...]: a device-resident dataset that the
    steps walk by themselves (``order``: optional int32 [nbatch] visiting order; a mask
    without the leading axis is shared by all minibatches, e.g. redrawn per step by a kernel
    in front).  The step counter lives on the device (``counters``).  Gradients land in
    ``net.dP``, the loss [I] in ``loss``; ``net.P`` holds the parameters after every step
    as the reference would (the look-ahead copy is ``PL``).  ``status`` is 2 after a step
    that met an empty region or one longer than ``max_rows``."""

    def __init__(self, net, X, R, Y, dropmask=None, order=None, max_rows=None):
        self.net = net
        dll = _lib.load()
        stacked = X.dim() == 2
        B = int(R.shape[-2])
        if max_rows is None:
            Rh = R.view(torch.int32).reshape(-1, 2).cpu().numpy().astype(np.int64)
            max_rows = int((Rh[:, 1] - Rh[:, 0]).max()) if len(Rh) else 1
        self.PL = torch.empty_like(net.P)
        self.loss = torch.zeros(net.I, dtype=torch.float32, device=net.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=net.dev)
        self.counters = torch.zeros(2, dtype=torch.int32, device=net.dev)
        self._keep = (X, R, Y, dropmask, order)
        a = _lib.c_ministep_args()
        a.nmodel, a.nfilt, a.m, a.ptype = net.I, net.nf // net.I, net.m, POOL_CODE[net.pool]
        a.hidden, a.loss_kind, a.strand_pairs, a.B = net.hidden, 1 if net.loss == "nll" else 0, int(net.strand_pairs), B
        a.max_rows, a.npos = max(1, int(max_rows)), int(X.shape[-1])
        a.X, a.X_stride = X.data_ptr(), X.stride(0) * X.element_size() if stacked else 0
        a.R, a.R_stride = R.data_ptr(), R.stride(0) * R.element_size() if R.dim() == 3 else 0
        a.Y, a.Y_stride = Y.data_ptr(), Y.stride(0) * Y.element_size() if Y.dim() == 3 else 0
        if dropmask is not None:
            a.dropmask, a.mask_stride = dropmask.data_ptr(), dropmask.stride(0) * dropmask.element_size() if dropmask.dim() == 3 else 0
        if stacked:
            a.counters, a.nbatch = self.counters.data_ptr(), int(X.shape[0])
            a.order = order.data_ptr() if order is not None else None
        a.P, a.PL, a.mP, a.dP = net.P.data_ptr(), self.PL.data_ptr(), net.mP.data_ptr(), net.dP.data_ptr()
        a.drate, a.mrate = net.drate.data_ptr(), net.mrate.data_ptr()
        off = {k: int(net.offsets[i]) for i, k in enumerate(net.names)}
        a.off_Wscan, a.off_bscan, a.off_W1, a.off_b1 = off["Wscan"], off["bscan"], off["W1"], off["b1"]
        a.off_W2, a.off_b2 = off.get("W2", 0), off.get("b2", 0)
        a.loss, a.status = self.loss.data_ptr(), self.status.data_ptr()
        self.args = a
        ok = all(t.is_contiguous() for t in (X, R, Y)) and X.dtype == torch.uint8 and Y.dtype == torch.float32
        self.supported = bool(ok and dll.db_ministep_supported(ctypes.byref(a)))
        self.scratch_bytes = int(dll.db_ministep_scratch_bytes(ctypes.byref(a))) if self.supported else 0

    def lookahead(self):
        """PL = P + mrate * mP: before the first step and after any change of P or mP
        made elsewhere (gradstep.cu:46-50)."""
        bind_stream()
        n = self.net
        _lib.load().db_ministep_lookahead(self.PL.data_ptr(), n.P.data_ptr(), n.mP.data_ptr(), n.mrate.data_ptr(), n.P.numel())

    def run(self):
        """Enqueues one step on the current stream."""
        bind_stream()
        n = self.net
        self.args.decay = n.decay.data_ptr() if (n.decay_on and n.decay is not None) else None
        _lib.load().db_ministep(ctypes.byref(self.args))
        return self.loss

    def capture(self, steps=1, prologue=None):
        """CUDA graph of the look-ahead refresh and ``steps`` consecutive steps
        (``prologue``: a callable that launches further kernels in front of every step,
        e.g. the draw of the dropout mask).  The scratch buffer is sized first: nothing may
        be allocated while a stream is captured.  The step counter is not touched."""
        _lib.load().db_reserve_scratch(self.scratch_bytes)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.lookahead()
            for _ in range(steps):
                if prologue is not None:
                    prologue()
                self.run()
        return graph
