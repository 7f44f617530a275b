"""Partitioning of the path over the GPUs of one box.

The path shards by independent units, as the reference does with one worker
process per device (code/libs/deepity/deepity/hpsearch.py:324-330,376;
code/libs/kangaroo/kangaroo/predict.py:488): sequences for scoring, models for
training.  No data-path collective is needed; the only exchange is the final
gather of the score shards (or of a per-model metric vector).
"""
import torch
import torch.distributed as dist


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
