"""Fused hot-path entry points (plain device pointers through the C ABI).

``scanpool`` is the chain  corr1ord -> bias -> rectify -> poolrgn  of a
DeepBind convolutional stage in one kernel; ``scanpool_bprop`` is its
backward pass.  Tensors are CUDA ``torch.Tensor`` (memory only).
"""
import torch

from . import _lib
from .smat import bind_stream

PT = {"max": 0, "avg": 1, "sum": 2, "all": 3}


def _dll():
    dll = _lib.load()
    bind_stream()
    return dll


def _ptr(t):
    return None if t is None else t.data_ptr()


def _check(t, dtype, name):
    if not (t.is_cuda and t.is_contiguous() and t.dtype == dtype):
        raise TypeError("%s must be a contiguous CUDA tensor of %s" % (name, dtype))


def scanpool(W, bias, X, R, ptype="max", relu=True, want_argmax=False, want_actmask=False):
    """W [4m, nf] f32, bias [nf] f32 or None, X [npos] uint8, R [nregion, 2] int32
    (uint32 bit pattern).  Returns (pooled, argmax, actmask): pooled f32
    [nregion, nf] (or [nregion, 2nf] interleaved max, mean for "all"); argmax int32
    (uint32 bit pattern) flat indices row*nf+f or None; actmask int16 words
    [npos, ceil(nf/16)] or None."""
    _check(W, torch.float32, "W"); _check(X, torch.uint8, "X"); _check(R, torch.int32, "R")
    if bias is not None:
        _check(bias, torch.float32, "bias")
    m, nf = W.shape[0] // 4, W.shape[1]
    nregion, npos = R.shape[0], X.numel()
    pooled = torch.empty((nregion, nf * (2 if ptype == "all" else 1)), dtype=torch.float32, device=W.device)
    argmax = torch.empty((nregion, nf), dtype=torch.int32, device=W.device) if (want_argmax and ptype in ("max", "all")) else None
    actmask = torch.empty((npos, (nf + 15) // 16), dtype=torch.int16, device=W.device) if want_actmask else None
    _dll().db_scanpool_fwd(_ptr(W), m, nf, _ptr(bias), int(bool(relu)), _ptr(X), npos, _ptr(R), nregion,
                           PT[ptype], _ptr(pooled), _ptr(argmax), _ptr(actmask))
    return pooled, argmax, actmask


def scanpool_bprop(m, nf, X, R, ptype, dpooled, argmax, actmask, dW_out=None, db_out=None):
    """Returns (dW [4m, nf], dbias [nf]) of the fused stage; ``dW_out`` / ``db_out``
    (contiguous f32) receive them in place, e.g. slices of a flat gradient vector."""
    _check(dpooled, torch.float32, "dpooled")
    dW = dW_out if dW_out is not None else torch.empty((4 * m, nf), dtype=torch.float32, device=dpooled.device)
    db = db_out if db_out is not None else torch.empty((nf,), dtype=torch.float32, device=dpooled.device)
    _check(dW, torch.float32, "dW_out"); _check(db, torch.float32, "db_out")
    assert dW.numel() == 4 * m * nf and db.numel() == nf
    _dll().db_scanpool_bwd(m, nf, _ptr(X), X.numel(), _ptr(R), R.shape[0], PT[ptype], _ptr(dpooled),
                           _ptr(argmax), _ptr(actmask), _ptr(dW), _ptr(db))
    return dW, db


def build_batch(seqs, padding, reverse_complement=False, device="cuda"):
    """A minibatch of sequence strings -> (X uint8 [npos], R int32 [nrow, 2]) on the
    device, laid out as kangaroo's ``_seqdata._pack`` does (data.py:274-334): the
    characters are uploaded once and translated, padded and (optionally)
    reverse-complemented by one kernel.  ``seqs`` may also be a pair
    (text uint8 tensor, offsets int32 tensor [nseq+1]) already on the device."""
    import numpy as np
    if isinstance(seqs, tuple):
        text, off = seqs
        _check(text, torch.uint8, "text"); _check(off, torch.int32, "offsets")
        nseq = off.numel() - 1
        total = int(off[-1].item() - off[0].item()) if nseq > 0 else 0
    else:
        nseq = len(seqs)
        raw = "".join(seqs).encode("latin-1")
        total = len(raw)
        lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=nseq)
        off_h = np.zeros(nseq + 1, dtype=np.int64)
        np.cumsum(lens, out=off_h[1:])
        text = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device) if total else torch.empty(0, dtype=torch.uint8, device=device)
        off = torch.from_numpy(off_h.astype(np.int32)).to(device)
    dll = _dll()
    rc = int(bool(reverse_complement))
    nbytes = dll.db_batch_bytes(nseq, total, padding, rc)
    if nbytes >= 2 ** 32:
        raise ValueError("a minibatch is addressed with 32-bit positions; split it")
    X = torch.empty(nbytes, dtype=torch.uint8, device=text.device)
    R = torch.empty((nseq * (2 if rc else 1), 2), dtype=torch.int32, device=text.device)
    dll.db_build_batch(_ptr(text), _ptr(off), nseq, padding, rc, _ptr(X), _ptr(R))
    return X, R


def _upload_text(seqs, device):
    import numpy as np
    nseq = len(seqs)
    raw = "".join(seqs).encode("latin-1")
    lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=nseq)
    off_h = np.zeros(nseq + 1, dtype=np.int64)
    np.cumsum(lens, out=off_h[1:])
    text = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device) if raw else torch.empty(0, dtype=torch.uint8, device=device)
    return text, torch.from_numpy(off_h.astype(np.int32)).to(device), lens


def window_counts(lens, windowsize, stride):
    """Windows per sequence in scan mode: every ``stride``-th start in the sequence
    padded with windowsize-1 'N' on both sides (predict.py:281-284)."""
    import numpy as np
    lens = np.asarray(lens, dtype=np.int64)
    return (np.maximum(1, lens + windowsize - 1) + stride - 1) // stride


def build_windows(seqs, windowsize, stride, padding, reverse_complement=False, device="cuda"):
    """Scan-mode minibatch of sequence strings: every window of every sequence as a
    row -> (X uint8, R int32 [nrow, 2], window_offsets int64 numpy [nseq+1]), built by
    one kernel from the uploaded characters (the reference expands the windows as
    Python strings, predict.py:270-285)."""
    import numpy as np
    if windowsize == 1 and any(len(s) == 0 for s in seqs):
        raise ValueError("scan mode with windows of one character needs non-empty sequences")
    text, off, lens = _upload_text(seqs, device)
    nwin = window_counts(lens, windowsize, stride)
    woff_h = np.zeros(len(seqs) + 1, dtype=np.int64)
    np.cumsum(nwin, out=woff_h[1:])
    total = int(woff_h[-1])
    dll = _dll()
    rc = int(bool(reverse_complement))
    nbytes = dll.db_batch_bytes(total, total * windowsize, padding, rc)
    if nbytes >= 2 ** 32:
        raise ValueError("a minibatch is addressed with 32-bit positions; split it")
    woff = torch.from_numpy(woff_h.astype(np.int32)).to(device)
    X = torch.empty(nbytes, dtype=torch.uint8, device=device)
    R = torch.empty((total * (2 if rc else 1), 2), dtype=torch.int32, device=device)
    dll.db_build_windows(_ptr(text), _ptr(off), _ptr(woff), len(seqs), total, windowsize, stride, padding, rc, _ptr(X), _ptr(R))
    return X, R, woff_h


class MinibatchFeed(object):
    """Device-resident dataset cut into ``nbatch`` equal minibatches, fetched by one
    launch per step (db_minibatch_fetch): ``pairs`` is a list of up to three
    (dataset tensor [nbatch, ...], step buffer [...]) pairs -- sequences, targets,
    dropout masks.  ``fetch()`` copies the next minibatch into the step buffers and
    advances the device-side step counter; captured into a CUDA graph in front of a
    training step, the whole loop replays without host work.  ``order`` (optional int32
    device tensor [nbatch]) gives the minibatch visited at each step of an epoch."""

    def __init__(self, pairs, order=None):
        assert 1 <= len(pairs) <= 3
        self.pairs = [(a.contiguous(), b) for a, b in pairs]
        self.nbatch = int(self.pairs[0][0].shape[0])
        for a, b in self.pairs:
            assert a.shape[0] == self.nbatch and a[0].numel() * a.element_size() == b.numel() * b.element_size()
            assert b.is_contiguous()
        self.order = order
        self.counters = torch.zeros(2, dtype=torch.int32, device=self.pairs[0][0].device)

    def fetch(self):
        bind_stream()
        args = []
        for k in range(3):
            if k < len(self.pairs):
                a, b = self.pairs[k]
                args += [_ptr(a), _ptr(b), b.numel() * b.element_size()]
            else:
                args += [None, None, 0]
        _dll().db_minibatch_fetch(_ptr(self.counters), _ptr(self.order) if self.order is not None else None, self.nbatch, *args)


TC_PRECISION = {"bf16": 1, "bf16x2": 2, "bf16x3": 3, "f16x2": 4, "f16": 5}
TC_PIECES = {1: 1, 2: 2, 3: 3, 4: 2, 5: 1}     # 16-bit operand pieces per weight = tensor-core passes


class TCWeights(object):
    """Filter bank prepared for the tensor-core scan: 16-bit operand tiles.

    ``precision``: "bf16", "bf16x2", "bf16x3" (1-3 bf16 pieces per weight: 8, 16, 24
    significant bits) or "f16", "f16x2" (1-2 f16 pieces of power-of-two prescaled
    weights: 11, 22 bits); the integers 1-5 of ``enum db_tc_precision`` also work."""

    def __init__(self, W, bias=None, precision="f16x2"):
        _check(W, torch.float32, "W")
        self.precision = TC_PRECISION[precision] if isinstance(precision, str) else int(precision)
        self.m, self.nf, self.nsplit = W.shape[0] // 4, W.shape[1], TC_PIECES[self.precision]
        self.bias = bias
        dll = _dll()
        nbytes = dll.db_tc_weights_bytes(self.m, self.nf, self.precision)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=W.device)
        dll.db_tc_prepare(_ptr(W), self.m, self.nf, self.precision, _ptr(self.buf))


def scanpool_tc(tcw, X, R, ptype="all", relu=True, headW=None, headB=None, want_pooled=None, check=True,
                scores_out=None, status=None):
    """Tensor-core scan + bias + rectify + pooling of a prepared filter bank.

    Returns (pooled, scores): pooled as :func:`scanpool` (or None), scores
    [nregion, nmodel] when a linear head (headW [(16|32)*nmodel], headB [nmodel])
    is given.  ``check`` reads the kernel's status word back (one sync);
    ``scores_out`` / ``status`` let a caller reuse its buffers (status must be a
    zeroed int32 tensor of one element)."""
    _check(X, torch.uint8, "X"); _check(R, torch.int32, "R")
    nregion, npos, nf = R.shape[0], X.numel(), tcw.nf
    if want_pooled is None:
        want_pooled = headW is None
    pooled = torch.empty((nregion, nf * (2 if ptype == "all" else 1)), dtype=torch.float32, device=X.device) if want_pooled else None
    nmodel = nf // 16 if headW is not None else 0
    scores = None
    if headW is not None:
        scores = scores_out if scores_out is not None else torch.empty((nregion, nmodel), dtype=torch.float32, device=X.device)
        _check(scores, torch.float32, "scores_out")
        assert tuple(scores.shape) == (nregion, nmodel)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=X.device)
    _dll().db_scanpool_tc(_ptr(tcw.buf), tcw.m, nf, tcw.precision, _ptr(tcw.bias), int(bool(relu)), _ptr(X), npos, _ptr(R),
                          nregion, PT[ptype], _ptr(pooled), _ptr(headW), _ptr(headB), nmodel, _ptr(scores), _ptr(status))
    if check:
        code = int(status.item())
        if code:
            raise _lib.SmatException("scanpool_tc(...) raised an exception\nRuntimeError: tensor-core scan failed: %s" %
                                     {1: "a device-side wait timed out", 3: "regions must ascend without overlap",
                                      4: "the filter bank holds an Inf or NaN weight"}.get(code, code))
    return pooled, scores
