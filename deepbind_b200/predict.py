"""Scoring driver with the semantics of ``kangaroo.predict``.

Direct mode scores every sequence once (predict.py:168-196); scan mode
(predict.py:262-345, 434-452) slides a window along each sequence, scores every
window as a sequence of its own and reports the maximum, mean and sum of each
sequence's prediction map.  All models of a :class:`DeepBindNet` are scored in
the same pass (the reference runs one worker process per model,
predict.py:466-508).  Batch assembly, window expansion, scan, pooling, head,
strand choice and the per-sequence reductions run on the device; the host only
uploads the characters.
"""
import numpy as np
import torch

from . import fused
from . import kangaroo_smat as ks
from . import smat as sm


def _score(net, X, R, reverse_complement):
    return net.score(X, R, strand_max=bool(reverse_complement))


def predict(net, seqs, scan=None, stride=1, reverse_complement=False, want_pmaps=False, max_windows=1 << 21):
    """Scores the sequence strings ``seqs`` with every model of ``net``.

    Returns a dict of CUDA tensors [nseq, I]: ``direct``; with ``scan`` = window
    size also ``max``, ``avg``, ``sum`` over each sequence's windows, and ``pmaps``
    (a list of [nwindow_b, I] tensors, one per sequence) if ``want_pmaps``.  With
    ``reverse_complement`` both strands are scored and the larger score is kept,
    the forward strand on ties (predict.py:145-164).  Sequences are processed in
    groups of at most ``max_windows`` windows."""
    seqs = list(seqs)
    pad = net.m - 1
    dev = net.dev
    X, R = fused.build_batch(seqs, pad, reverse_complement, device=dev)
    out = {"direct": _score(net, X, R, reverse_complement)}
    if not scan:
        return out
    lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=len(seqs))
    nwin = fused.window_counts(lens, scan, stride)
    if int(nwin.max(initial=0)) > max_windows:
        raise ValueError("a sequence has more windows than max_windows")
    red = {"max": [], "avg": [], "sum": []}
    pmaps = []
    lo = 0
    while lo < len(seqs):
        hi, total = lo, 0
        while hi < len(seqs) and total + int(nwin[hi]) <= max_windows:
            total += int(nwin[hi]); hi += 1
        Xw, Rw, woff = fused.build_windows(seqs[lo:hi], scan, stride, pad, reverse_complement, device=dev)
        Z = _score(net, Xw, Rw, reverse_complement).contiguous()            # [windows, I]: the prediction maps, stacked
        # per-sequence reductions = region pooling over the rows of Z
        regions = sm.asarray(np.stack([woff[:-1], woff[1:]], axis=1).astype(np.uint32))
        Zs = sm.sarray(Z, np.float32)
        for kind in red:
            red[kind].append(ks.poolrgn(Zs, regions, kind)[0].tensor)
        if want_pmaps:
            pmaps.extend(Z[int(woff[i]):int(woff[i + 1])] for i in range(hi - lo))
        lo = hi
    for kind in red:
        out[kind] = torch.cat(red[kind]) if red[kind] else torch.empty((0, net.I), dtype=torch.float32, device=dev)
    if want_pmaps:
        out["pmaps"] = pmaps
    return out


def gradient_maps(net, seqs, reverse_complement=False, batchsize=2048):
    """Gradient maps of direct-mode scoring (predict.py:198-265): for every sequence the
    [len, 4] gradient of the fed-back output with respect to the four channels of each
    position (``DeepBindNet.input_gradients``), batch by batch of ``batchsize`` sequences
    as the reference evaluates them.  With ``reverse_complement`` the map of the stronger
    strand is kept (the forward one on ties), in that strand's own coordinates.

    Returns (Z [nseq, I] CUDA tensor, maps: list of numpy [len_b, 4], strands: numpy int8
    [nseq], 0 = forward, 1 = reverse complement).  Several models: the fed-back gradients
    of all models add up in dX, as they do in the reference's shared input plug."""
    seqs = list(seqs)
    pad = net.m - 1
    rc = bool(reverse_complement)
    Zs, maps, strands = [], [], []
    for lo in range(0, len(seqs), batchsize):
        chunk = seqs[lo:lo + batchsize]
        X, R = fused.build_batch(chunk, pad, rc, device=net.dev)
        Z, dX = net.input_gradients(X, R, strand_max=rc)
        Rh = R.cpu().numpy().view(np.uint32)
        dXh = dX.cpu().numpy()
        if rc:
            z = Z.view(-1, 2, net.I)
            fwd = (z[:, 0, 0] >= z[:, 1, 0]).cpu().numpy()          # the first model's outputs choose the strand
            Zs.append(torch.where(z[:, 0] >= z[:, 1], z[:, 0], z[:, 1]))
            for b in range(len(chunk)):
                r = 2 * b + (0 if fwd[b] else 1)
                maps.append(dXh[Rh[r, 0] + pad:Rh[r, 1]].copy())
                strands.append(0 if fwd[b] else 1)
        else:
            Zs.append(Z)
            for b in range(len(chunk)):
                maps.append(dXh[Rh[b, 0] + pad:Rh[b, 1]].copy())
                strands.append(0)
    return torch.cat(Zs), maps, np.asarray(strands, np.int8)


_ORD = np.full(256, 255, np.uint8)
for _k, _c in enumerate("ACGT"):
    _ORD[ord(_c)] = _k
    _ORD[ord(_c.lower())] = _k
_ORD[ord("U")] = _ORD[ord("u")] = 3


def mutation_maps(net, seqs, reverse_complement=False):
    """Mutation maps of kangaroo.predict (``want_gmaps="finite_diff"``, predict.py:208-250):
    every position of every sequence is set to each of the four bases in turn, the mutant
    is scored like the sequence itself (both strands and the larger score with
    ``reverse_complement``), and the map holds mtZ - Z, set to 0 where neither score is
    positive.  The 4 * len mutants of a sequence are laid out as one batch directly in
    ordinal form (no strings) and scored by the fused scan kernel in one pass.

    Returns (Z [nseq, I] numpy, maps: list of numpy [len_b, 4, I])."""
    pad = net.m - 1
    rc = bool(reverse_complement)
    Zs, maps = [], []
    for s in seqs:
        o = _ORD[np.frombuffer(s.encode("latin-1"), np.uint8)]
        L = len(o)
        rows = np.tile(o, (4 * L + 1, 1))                        # row 0: the sequence itself
        idx = np.arange(L)
        for j in range(4):
            rows[1 + 4 * idx + j, idx] = j
        if rc:
            rev = rows[:, ::-1].copy()
            acgt = rev < 4
            rev[acgt] = 3 - rev[acgt]
            rows = np.stack([rows, rev], 1).reshape(-1, L)       # forward, reverse complement, forward, ...
        n = rows.shape[0]
        Xh = np.full((n, pad + L), 255, np.uint8)
        Xh[:, pad:] = rows
        Xh = np.concatenate([Xh.ravel(), np.full(pad, 255, np.uint8)])
        Rh = (np.arange(n, dtype=np.int64)[:, None] * (pad + L) + np.array([0, pad + L])).astype(np.int32)
        Z = net.score(torch.from_numpy(Xh).to(net.dev), torch.from_numpy(Rh).to(net.dev), strand_max=rc).cpu().numpy()
        z0, mt = Z[0], Z[1:].reshape(L, 4, net.I)
        d = mt - z0
        d *= np.maximum(0, np.sign(np.maximum(z0, mt)))
        Zs.append(z0)
        maps.append(d)
    return np.stack(Zs), maps
