"""The N>1 path on CPU: two gloo ranks shard a batch by sequence, score their
shards (with the CPU oracle standing in for the kernel) and gather the score
shards; the result must equal the single-process scores.  Also a rank that fails
on the host is reported to its peer through the store, without any GPU."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir, fail_rank):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepbind_b200 import shard, synth
    from oracle import oracle as orc
    orc.set_num_threads(1)
    m, I, nseq = 16, 3, 37                                   # 37 does not divide by 2: ragged shards
    X, R = synth.ragged_batch(nseq, 20, 60, m, seed=5, n_frac=0.05)
    p = synth.model_params(I, m, 6, "all")
    lo, hi = shard.shard_range(nseq, rank, world)
    store = dist.distributed_c10d._get_default_store()
    try:
        if rank == fail_rank:
            raise RuntimeError("injected host failure")
        row_lo, row_hi = shard.region_shard(R, lo, hi, m)
        Xs = X[row_lo:row_hi]
        Rs = (R[lo:hi].astype(np.int64) - row_lo).astype(np.uint32)
        local = torch.from_numpy(orc.score_net(p, Xs, Rs, "all", I))
        store.set("status_%d" % rank, "ok")
    except Exception as e:                                   # a failed rank tells its peers before leaving
        store.set("status_%d" % rank, "error: %s" % e)
        local = None
    statuses = [store.get("status_%d" % r).decode() for r in range(world)]
    if any(s != "ok" for s in statuses):
        np.save(os.path.join(out_dir, "status_%d.npy" % rank), np.array(statuses))
        dist.destroy_process_group()
        return
    full = shard.gather_scores(local)
    np.save(os.path.join(out_dir, "scores_%d.npy" % rank), full.numpy())
    dist.destroy_process_group()


def _run(tmp_path, fail_rank=-1):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path), fail_rank), nprocs=2, join=True)


def test_shard_helpers():
    from deepbind_b200 import shard
    assert [shard.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert shard.shard_range(0, 0, 2) == (0, 0)
    assert shard.shard_models(90, 3, 8) == list(range(3, 90, 8))
    assert sorted(sum((shard.shard_models(90, r, 8) for r in range(8)), [])) == list(range(90))


def test_two_ranks_score_and_gather(tmp_path):
    sys.path.insert(0, ROOT)
    from deepbind_b200 import synth
    from oracle import oracle as orc
    _run(tmp_path)
    X, R = synth.ragged_batch(37, 20, 60, 16, seed=5, n_frac=0.05)
    want = orc.score_net(synth.model_params(3, 16, 6, "all"), X, R, "all", 3)
    for r in range(2):
        got = np.load(os.path.join(str(tmp_path), "scores_%d.npy" % r))
        assert got.shape == want.shape
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)


def test_host_failure_reaches_the_peer(tmp_path):
    _run(tmp_path, fail_rank=1)
    for r in range(2):
        st = np.load(os.path.join(str(tmp_path), "status_%d.npy" % r))
        assert st[0] == "ok" and st[1].startswith("error: injected host failure")


def _chunk_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepbind_b200 import shard
    n, I, nchunk = 10, 3, 3                                  # chunks of 4, 3, 3 rows
    src = torch.arange(n * I, dtype=torch.float32).reshape(n, I) + 1000 * rank
    local = torch.zeros_like(src)
    calls = []

    def produce(lo, hi):                                     # the "kernel": fills one chunk of the shard
        calls.append((lo, hi))
        local[lo:hi] = src[lo:hi]
    outs = [torch.empty((world * (hi - lo), I)) for lo, hi in (shard.shard_range(n, c, nchunk) for c in range(nchunk))]
    shard.chunked_gather(produce, local, outs)
    full = shard.gathered_rows(outs, n, world)
    np.save(os.path.join(out_dir, "chunked_%d.npy" % rank), full.numpy())
    np.save(os.path.join(out_dir, "calls_%d.npy" % rank), np.array(calls))
    dist.destroy_process_group()


def test_chunked_gather_overlap_order(tmp_path):
    """Chunk-by-chunk gather of two ranks' shards gives the rank-major matrix."""
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_chunk_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    want = np.concatenate([np.arange(30, dtype=np.float32).reshape(10, 3) + 1000 * r for r in range(2)])
    for r in range(2):
        assert np.array_equal(np.load(os.path.join(str(tmp_path), "chunked_%d.npy" % r)), want)
        assert np.load(os.path.join(str(tmp_path), "calls_%d.npy" % r)).tolist() == [[0, 4], [4, 7], [7, 10]]
