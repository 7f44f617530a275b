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


def _predict_worker(rank, world, port, out_dir):
    """predict(..., group=) on two gloo ranks; the device kernels are replaced by the CPU
    oracle (batch assembly and scoring), so what runs here is the package's sharding and
    gathering of the sequence list."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepbind_b200 import fused, predict as P, synth
    from oracle import oracle as orc
    orc.set_num_threads(1)
    m, I = 16, 2
    params = synth.model_params(I, m, 6, "max")

    def build_batch(seqs, padding, reverse_complement=False, device=None):
        X, R = orc.asbatch(seqs, padding, reverse_complement)
        return torch.from_numpy(X), torch.from_numpy(R.view(np.int32))

    class Net(object):
        dev = torch.device("cpu")

        def __init__(self):
            self.I, self.m = I, m

        def score(self, X, R, strand_max=False):
            return torch.from_numpy(orc.score_net(params, X.numpy(), R.numpy().view(np.uint32), "max", I, strand_max=strand_max))
    fused.build_batch = build_batch
    rng = np.random.default_rng(3)
    seqs = ["".join(rng.choice(list("ACGT"), size=int(n))) for n in rng.integers(16, 50, size=11)]     # 11 = 6 + 5 per rank
    for rc in (False, True):
        got = P.predict(Net(), seqs, reverse_complement=rc, group="world")
        np.save(os.path.join(out_dir, "predict_%d_%d.npy" % (rank, rc)), got["direct"].numpy())
    # one rank without any sequence still takes part in the gather
    got = P.predict(Net(), seqs[:1], group=dist.group.WORLD)
    np.save(os.path.join(out_dir, "predict_one_%d.npy" % rank), got["direct"].numpy())
    dist.destroy_process_group()


def test_predict_shards_sequences_over_the_group(tmp_path):
    sys.path.insert(0, ROOT)
    from deepbind_b200 import synth
    from oracle import oracle as orc
    port = 33500 + (os.getpid() % 2000)
    mp.spawn(_predict_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    rng = np.random.default_rng(3)
    seqs = ["".join(rng.choice(list("ACGT"), size=int(n))) for n in rng.integers(16, 50, size=11)]
    params = synth.model_params(2, 16, 6, "max")
    for rc in (False, True):
        X, R = orc.asbatch(seqs, 15, rc)
        want = orc.score_net(params, X, R, "max", 2, strand_max=rc)
        for r in range(2):
            got = np.load(os.path.join(str(tmp_path), "predict_%d_%d.npy" % (r, rc)))
            assert got.shape == (11, 2)
            np.testing.assert_array_equal(got, want)
    X, R = orc.asbatch(seqs[:1], 15, False)
    for r in range(2):
        np.testing.assert_array_equal(np.load(os.path.join(str(tmp_path), "predict_one_%d.npy" % r)),
                                      orc.score_net(params, X, R, "max", 2))


def _records_worker(rank, world, port, out_dir):
    """The exchange of calibrate(..., group=): samples dealt round robin, per-rank record
    dictionaries merged on every rank, per-trial values dealt back into trial order."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepbind_b200 import shard
    ncalib = 7
    mine = shard.shard_models(ncalib, rank, world)
    records = {(s, step): {"sample": s, "step": step, "folds": [s + 0.1 * step]} for s in mine for step in (10, 20)}
    merged = {k: v for part in shard.gather_objects(records) for k, v in part.items()}
    vals = shard.deal_back(shard.gather_objects([10.0 * s for s in mine]), ncalib, world)
    ok = shard.checksum_agrees(torch.arange(5.0) + 1) and not shard.checksum_agrees(torch.arange(5.0) + rank)
    np.save(os.path.join(out_dir, "records_%d.npy" % rank), np.array([sorted(merged) == [(s, st) for s in range(ncalib) for st in (10, 20)],
                                                                      vals == [10.0 * s for s in range(ncalib)], ok]))
    dist.destroy_process_group()


def test_calibration_records_are_merged_on_every_rank(tmp_path):
    port = 35500 + (os.getpid() % 2000)
    mp.spawn(_records_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert np.load(os.path.join(str(tmp_path), "records_%d.npy" % r)).all()


def test_instances_cut_out_of_a_parameter_set():
    """cfg.select_instances keeps exactly the columns / row blocks of the chosen instances."""
    sys.path.insert(0, ROOT)
    from deepbind_b200 import cfg
    I, F, m, H = 5, 16, 4, 3
    rng = np.random.default_rng(0)
    p = {"Wscan": rng.standard_normal((4 * m, I * F)), "bscan": rng.standard_normal(I * F),
         "W1": rng.standard_normal((I * 2 * F, H)), "b1": rng.standard_normal(I * H),
         "W2": rng.standard_normal((I * H, 1)), "b2": rng.standard_normal(I)}
    ids = np.array([3, 0])
    q = cfg.select_instances(p, ids, I)
    assert np.array_equal(q["Wscan"], np.concatenate([p["Wscan"][:, 3 * F:4 * F], p["Wscan"][:, :F]], axis=1))
    assert np.array_equal(q["bscan"], np.concatenate([p["bscan"][3 * F:4 * F], p["bscan"][:F]]))
    assert np.array_equal(q["W1"], np.concatenate([p["W1"][3 * 2 * F:4 * 2 * F], p["W1"][:2 * F]]))
    assert np.array_equal(q["b1"], np.concatenate([p["b1"][3 * H:4 * H], p["b1"][:H]]))
    assert np.array_equal(q["W2"], np.concatenate([p["W2"][3 * H:4 * H], p["W2"][:H]]))
    assert np.array_equal(q["b2"], p["b2"][[3, 0]])
