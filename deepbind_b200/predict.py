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

from . import fused, shard
from . import kangaroo_smat as ks
from . import smat as sm


def _score(net, X, R, reverse_complement, precision=None):
    if precision is None:
        return net.score(X, R, strand_max=bool(reverse_complement))
    tcw = getattr(net, "_tcw", None)
    if tcw is None or tcw.precision != fused.TC_PRECISION[precision]:
        net.prepare_tc(precision)
    return net.score_tc(X, R, strand_max=bool(reverse_complement))


def predict(net, seqs, scan=None, stride=1, reverse_complement=False, want_pmaps=False, max_windows=1 << 21, group=None,
            precision=None):
    """Scores the sequence strings ``seqs`` with every model of ``net``.

    Returns a dict of CUDA tensors [nseq, I]: ``direct``; with ``scan`` = window
    size also ``max``, ``avg``, ``sum`` over each sequence's windows, and ``pmaps``
    (a list of [nwindow_b, I] tensors, one per sequence) if ``want_pmaps``.  With
    ``reverse_complement`` both strands are scored and the larger score is kept,
    the forward strand on ties (predict.py:145-164).  Sequences are processed in
    groups of at most ``max_windows`` windows.

    ``precision``: None scores with the exact FP32 kernels (pooled values bit-identical to the
    operator-by-operator chain); "f16x2" or "bf16x3" with the tensor-core scan at fp32 grade
    (exact products, another summation order: within 1e-5 of the exact scores, typically
    below 1e-6), "f16" / "bf16" with one 16-bit piece per weight (5e-4 / 2e-3 of the largest
    activation).  The weights are prepared once per ``net`` and precision; call
    ``net.prepare_tc`` again after changing them.

    ``group`` (a torch.distributed process group, or "world" for the default one; one
    process per GPU, every rank holding the same ``net`` and ``seqs``): the sequences
    are split into contiguous shards, one per rank, as the reference splits its work
    over one process per device (predict.py:484-492); every rank scores its shard and
    the score shards are all-gathered, so every rank returns all rows.  ``pmaps`` stay
    those of the rank's own shard (``shard.shard_range(len(seqs), rank, world)``)."""
    seqs = list(seqs)
    if group is not None:
        grp = None if (isinstance(group, str) and group == "world") else group
        rank, world = shard.rank_world(grp)
        if world > 1:
            lo, hi = shard.shard_range(len(seqs), rank, world)
            mine = predict(net, seqs[lo:hi], scan, stride, reverse_complement, want_pmaps, max_windows, precision=precision) if hi > lo else \
                {k: torch.empty((0, net.I), dtype=torch.float32, device=net.dev) for k in (("direct", "max", "avg", "sum") if scan else ("direct",))}
            out = {k: shard.gather_scores(v.contiguous(), grp) for k, v in mine.items() if k != "pmaps"}
            if want_pmaps and scan:
                out["pmaps"] = mine.get("pmaps", [])
            return out
    pad = net.m - 1
    dev = net.dev
    X, R = fused.build_batch(seqs, pad, reverse_complement, device=dev)
    out = {"direct": _score(net, X, R, reverse_complement, precision)}
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
        Z = _score(net, Xw, Rw, reverse_complement, precision).contiguous() # [windows, I]: the prediction maps, stacked
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


class ShardedScorer(object):
    """Scores a device-resident ordinal batch over the ranks of a process group with the
    tensor-core scan: every rank scans its own regions in ``nchunk`` pieces and each
    piece's all-gather (NCCL, asynchronous) runs while the next piece is scanned, so
    that every rank ends up with the scores of all ranks' sequences -- the scoring path
    of kangaroo.predict fanned out over the devices of one box (predict.py:484-492)
    with the gather overlapped.  Buffers are allocated once and reused by every call.

    ``gather="peer"`` does without the collective: the gathered matrix of every rank
    lies in symmetric memory (torch.distributed._symmetric_memory, every rank's buffer
    mapped into every process), the scan kernel stores each score straight into all of
    them over NVLink while it runs (``db_scanpool_tc_peers``), one launch scans the whole
    shard, and a one-element all-reduce afterwards is the barrier that tells every rank
    that all stores have landed.  No second pass over the scores, no NCCL kernels
    competing with the scan for SMs.  Only plain peer stores are used (no multicast).

    ``net``: a DeepBindNet with the in-kernel linear head (no hidden layer) whose
    tensor-core weights were prepared; ``nseq``: regions per rank (the same on every
    rank)."""

    def __init__(self, net, nseq, group=None, nchunk=8, gather="nccl"):
        import torch.distributed as dist
        self.net, self.group, self.nseq = net, group, int(nseq)
        self.rank, self.world = shard.rank_world(group)
        self.nchunk = max(1, min(int(nchunk), self.nseq))
        self.scores = torch.empty((self.nseq, net.I), dtype=torch.float32, device=net.dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=net.dev)
        self.gathered = self.chunks = self._peers = None
        if gather not in ("nccl", "peer"):
            raise ValueError("gather must be 'nccl' or 'peer', got %r" % (gather,))
        self.gather = gather if self.world > 1 else "nccl"
        if self.gather == "peer":
            import ctypes
            import os
            # the kernel uses plain peer stores; without an NVSwitch multicast binding a rank
            # that leaves early cannot disturb the others' buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            if self.world > 8:
                raise ValueError("the peer gather serves at most 8 ranks (one box)")
            self.gathered = symm.empty((self.nseq * self.world, net.I), dtype=torch.float32, device=net.dev)
            self._symm = symm.rendezvous(self.gathered, dist.group.WORLD if group is None else group)
            ptrs = [int(q) for q in self._symm.buffer_ptrs]
            if len(ptrs) != self.world or ptrs[self.rank] != self.gathered.data_ptr():
                raise RuntimeError("symmetric memory rendezvous returned an unexpected buffer table")
            self._peers = (ctypes.c_void_p * self.world)(*ptrs)
            self._flag = torch.zeros(1, dtype=torch.int32, device=net.dev)
            self.scores = self.gathered[self.rank * self.nseq:(self.rank + 1) * self.nseq]
        elif self.world > 1:
            self.gathered = torch.empty((self.nseq * self.world, net.I), dtype=torch.float32, device=net.dev)
            self.chunks = [self.gathered[self.world * lo:self.world * hi] for lo, hi in
                           (shard.shard_range(self.nseq, c, self.nchunk) for c in range(self.nchunk))]
        self._dist = dist

    def run(self, X, R):
        """Enqueues scan and gathers of this rank's batch (X ordinal buffer, R its
        ``nseq`` regions); returns the local score shard.  Call :meth:`check` after a
        synchronisation to learn of a failed scan."""
        net = self.net

        def rows(lo, hi):
            net.score_tc(X, R[lo:hi], check=False, out=self.scores[lo:hi], status=self.status)
        if self.world == 1:
            rows(0, self.nseq)
        elif self.gather == "peer":
            self._scan_to_peers(lambda: rows(0, self.nseq), 0)
            self._peer_barrier()
        else:
            shard.chunked_gather(rows, self.scores, self.chunks, self.group)
        return self.scores

    def _scan_to_peers(self, launch, row_lo):
        """Runs ``launch`` (scans that write rows row_lo.. of this rank's shard) with the
        peer stores switched on; the scan's own output is its rows of this rank's
        gathered matrix, the stores go to the other ranks' copies."""
        from ._lib import load as dll
        others = [q for r, q in enumerate(self._peers) if r != self.rank]
        tab = (type(self._peers)._type_ * len(others))(*others)
        dll().db_scanpool_tc_peers(tab, len(others), self.rank * self.nseq + row_lo)
        try:
            launch()
        finally:
            dll().db_scanpool_tc_peers(None, 0, 0)

    def _peer_barrier(self):
        """Stream-ordered barrier: the one-element all-reduce of a rank completes only
        after every rank's scan, enqueued before it, has finished."""
        self._dist.all_reduce(self._flag, group=self.group)

    def run_host(self, X_host, R_host, out_host, dev_bufs=None, wait=True):
        """The same from (pinned) host buffers to (pinned) host scores of this rank's
        shard: upload, scan and read-back are pipelined piece by piece
        (``DeepBindNet.predict_host``) and, with several ranks, every piece's all-gather
        starts as soon as the piece is enqueued.  Synchronises before it returns, unless
        ``wait=False`` (one rank, or the peer gather): then the call returns once everything
        is enqueued, the next call's uploads and scans overlap this call's last read-backs
        piece by piece, and :meth:`wait_host` synchronises and reports a failed scan."""
        if dev_bufs is None:
            dev_bufs = (torch.empty(X_host.shape, dtype=torch.uint8, device=self.net.dev),
                        torch.empty(R_host.shape, dtype=torch.int32, device=self.net.dev), self.scores)
        works = []
        if self.gather == "peer":
            from ._lib import load as dll
            others = [q for r, q in enumerate(self._peers) if r != self.rank]
            tab = (type(self._peers)._type_ * len(others))(*others)

            def piece_rows(lo, hi):              # predict_host calls this before it enqueues piece lo..hi
                dll().db_scanpool_tc_peers(tab, len(others), self.rank * self.nseq + lo)
            try:
                self.net.predict_host(X_host, R_host, out_host, dev_bufs=(dev_bufs[0], dev_bufs[1], self.scores), tc=True,
                                      npiece=self.nchunk, before_piece=piece_rows, wait=wait)
            finally:
                dll().db_scanpool_tc_peers(None, 0, 0)
            self._peer_barrier()
            if wait:
                torch.cuda.current_stream().synchronize()
            return out_host

        def gather_piece(lo, hi):
            c = len(works)
            works.append(self._dist.all_gather_into_tensor(self.chunks[c], self.scores[lo:hi], group=self.group, async_op=True))
        self.net.predict_host(X_host, R_host, out_host, dev_bufs=(dev_bufs[0], dev_bufs[1], self.scores), tc=True,
                              npiece=self.nchunk, on_piece=gather_piece if self.world > 1 else None,
                              wait=wait or self.world > 1)
        if self.world > 1 and not works:         # a batch too small for the pipelined path: gather it now
            shard.chunked_gather(lambda lo, hi: None, self.scores, self.chunks, self.group)
        for w in works:
            w.wait()
        if self.world > 1:
            torch.cuda.current_stream().synchronize()
        return out_host

    def wait_host(self):
        """Completes the :meth:`run_host` calls made with ``wait=False``."""
        self.net.predict_host_wait()
        torch.cuda.current_stream().synchronize()

    def check(self):
        st = int(self.status.item())
        if st:
            self.status.zero_()
            raise RuntimeError("tensor-core scan failed on rank %d (status %d)" % (self.rank, st))

    def all_scores(self):
        """[world * nseq, I] in rank-major row order (a copy out of the chunk buffers)."""
        if self.world == 1:
            return self.scores
        if self.gather == "peer":
            return self.gathered
        return shard.gathered_rows(self.chunks, self.nseq, self.world)

    def verify(self):
        """After a synchronised :meth:`run`: this rank's rows of the gathered matrix
        equal its own shard, and all ranks hold the same matrix (checksums agree)."""
        if self.world == 1:
            return True
        full = self.all_scores()
        own = torch.equal(full[self.rank * self.nseq:(self.rank + 1) * self.nseq], self.scores)
        ok = torch.tensor([1 if own else 0], device=self.scores.device)
        self._dist.all_reduce(ok, op=self._dist.ReduceOp.MIN, group=self.group)
        return bool(ok.item()) and shard.checksum_agrees(full, self.group)
