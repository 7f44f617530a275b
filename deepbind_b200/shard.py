"""Partitioning of the path over the GPUs of one box.

The path shards by independent units, as the reference does with one worker
process per device (code/libs/deepity/deepity/hpsearch.py:324-330,376;
code/libs/kangaroo/kangaroo/predict.py:488): sequences for scoring, models for
training.  No data-path collective is needed; the only exchange is the final
gather of the score shards (or of a per-model metric vector).
"""
import torch
import torch.distributed as dist


def rank_world(group=None):
    """(rank, world) of this process in ``group``; (0, 1) when no process group is in
    use (``group`` None and torch.distributed not initialised)."""
    if group is None and not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def shard_range(n, rank, world):
    """Contiguous shard [lo, hi) of n units for `rank`; sizes differ by at most one."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_models(nmodel, rank, world):
    """Model ids trained by `rank`: round robin, so that hyper-parameter draws of
    different cost spread evenly (hypertrain hands out samples the same way)."""
    return list(range(rank, nmodel, world))


def region_shard(R, lo, hi, m):
    """Rows of the ordinal buffer a shard of regions needs: (row_lo, row_hi) such that
    X[row_lo:row_hi] holds regions lo..hi-1 and the m-1 bytes the last window reads."""
    row_lo = int(R[lo, 0])
    row_hi = int(R[hi - 1, 1]) + m - 1
    return row_lo, row_hi


def chunked_gather(produce, local, out_chunks, group=None):
    """Computes a score shard in chunks and gathers each chunk while the next one is
    being computed.

    ``produce(lo, hi)`` enqueues, on the current stream, the work that fills
    ``local[lo:hi]``; ``out_chunks[c]`` ([world * rows_c, ...], rows_c from
    ``shard_range(len(local), c, len(out_chunks))``) receives chunk c of every rank,
    rank-major.  Each all-gather is started asynchronously right after its chunk
    was enqueued, so on NCCL it waits for that chunk only and overlaps the chunks
    that follow; the current stream waits for all of them at the end.
    :func:`gathered_rows` puts the chunks back into rank-major row order."""
    nchunk, n = len(out_chunks), local.shape[0]
    works = []
    for c in range(nchunk):
        lo, hi = shard_range(n, c, nchunk)
        produce(lo, hi)
        works.append(dist.all_gather_into_tensor(out_chunks[c], local[lo:hi], group=group, async_op=True))
    for w in works:
        w.wait()


def gathered_rows(out_chunks, n, world):
    """[world * n, ...] in rank-major row order from the chunk-major buffers of
    :func:`chunked_gather` (a copy; scoring code can also index the chunks directly:
    row i of rank r lies in chunk c at row r * rows_c + (i - lo_c))."""
    nchunk = len(out_chunks)
    parts = []
    for r in range(world):
        for c in range(nchunk):
            lo, hi = shard_range(n, c, nchunk)
            parts.append(out_chunks[c][r * (hi - lo):(r + 1) * (hi - lo)])
    return torch.cat(parts)


def gather_scores(local, group=None):
    """All ranks' score shards [n_r, I] -> [sum n_r, I] on every rank.  Shards may
    differ in length by one row (shard_range); shorter ones are padded for the
    collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    n = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    sizes = [torch.zeros_like(n) for _ in range(world)]
    dist.all_gather(sizes, n, group=group)
    sizes = [int(s.item()) for s in sizes]
    nmax = max(sizes)
    padded = local
    if local.shape[0] < nmax:
        padded = torch.cat([local, local.new_zeros((nmax - local.shape[0],) + tuple(local.shape[1:]))])
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded.contiguous(), group=group)
    return torch.cat([o[:s] for o, s in zip(out, sizes)])


def gather_objects(local, group=None):
    """Every rank's picklable ``local`` object -> the list of all of them, rank order,
    on every rank (host-side bookkeeping such as calibration records)."""
    rank, world = rank_world(group)
    if world == 1:
        return [local]
    out = [None] * world
    dist.all_gather_object(out, local, group=group)
    return out


def deal_back(per_rank_lists, n, world):
    """Inverse of :func:`shard_models` for results: ``per_rank_lists[r][i]`` belongs to
    unit ``r + i * world``; returns the n results in unit order."""
    out = [None] * n
    for r, lst in enumerate(per_rank_lists):
        ids = shard_models(n, r, world)
        assert len(lst) == len(ids), "rank %d returned %d results for %d units" % (r, len(lst), len(ids))
        for i, v in zip(ids, lst):
            out[i] = v
    return out


def checksum_agrees(t, group=None):
    """True on every rank iff all ranks hold the same float tensor ``t`` up to its
    float64 sum and sum of squares (a cheap check that a gather gave every rank the
    same matrix; outside any timed region)."""
    rank, world = rank_world(group)
    c = torch.stack([t.double().sum(), (t.double() ** 2).sum()])
    if world == 1:
        return True
    lo, hi = c.clone(), c.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    return bool(torch.equal(lo, hi))
