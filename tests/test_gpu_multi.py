"""The package's multi-GPU paths on real devices: one process per GPU over NCCL, spawned
from the test.  Needs at least two GPUs (skipped otherwise).  Sequences are sharded for
scoring, hyper-parameter samples for calibration; nothing but score shards, host records
and one model's parameters crosses NVLink.  NVLS is switched off for these short-lived
ranks."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _init(rank, world, port):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    return torch, dist


def _scorer_worker(rank, world, port, out_dir):
    torch, dist = _init(rank, world, port)
    from deepbind_b200 import synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import ShardedScorer, predict
    m, I, nseq = 24, 16, 40000
    net = DeepBindNet(synth.model_params(I, m, 7, "all"), I, "all")
    net.prepare_tc("f16x2")
    Xh, Rh = synth.uniform_batch(nseq, 101, m, seed=100 + rank)
    X, R = torch.from_numpy(Xh).cuda(), torch.from_numpy(Rh.view(np.int32)).cuda()
    sc = ShardedScorer(net, nseq, nchunk=5)
    sc.run(X, R)
    torch.cuda.synchronize()
    sc.check()
    ok = sc.verify()
    full = sc.all_scores()
    # host-to-host form: same scores, and the gather still reaches every rank
    X_host, R_host = torch.from_numpy(Xh).pin_memory(), torch.from_numpy(Rh.view(np.int32)).pin_memory()
    out_host = torch.empty((nseq, I), dtype=torch.float32).pin_memory()
    sc.run_host(X_host, R_host, out_host)
    ok = ok and sc.verify() and bool(torch.equal(out_host, sc.scores.cpu()))
    # every rank scores the other rank's batch alone and compares with what it was sent
    other = 1 - rank
    Xo, Ro = synth.uniform_batch(nseq, 101, m, seed=100 + other)
    want = net.score_tc(torch.from_numpy(Xo).cuda(), torch.from_numpy(Ro.view(np.int32)).cuda())
    ok = ok and float((full[other * nseq:(other + 1) * nseq] - want).abs().max()) <= 1e-6 * float(want.abs().max())
    # the gather done by the scan kernel itself (peer stores into symmetric memory): same matrix
    sp = ShardedScorer(net, nseq, nchunk=5, gather="peer")
    sp.run(X, R)
    torch.cuda.synchronize()
    sp.check()
    ok = ok and sp.verify() and bool(torch.equal(sp.all_scores(), full))
    sp.gathered.zero_()
    torch.cuda.synchronize(); dist.barrier()
    out_host.zero_()
    sp.run_host(X_host, R_host, out_host)
    ok = ok and sp.verify() and bool(torch.equal(sp.all_scores(), full)) and bool(torch.equal(out_host, sp.scores.cpu()))
    # predict() over the group: every rank gets all rows
    rng = np.random.default_rng(5)
    seqs = ["".join(rng.choice(list("ACGT"), size=int(n))) for n in rng.integers(30, 90, size=101)]
    net2 = DeepBindNet(synth.model_params(3, m, 9, "max"), 3, "max")
    got = predict(net2, seqs, reverse_complement=True, group="world")["direct"]
    alone = predict(net2, seqs, reverse_complement=True)["direct"]
    ok = ok and bool(torch.equal(got, alone))
    np.save(os.path.join(out_dir, "scorer_%d.npy" % rank), np.array([ok]))
    dist.destroy_process_group()


def test_sharded_scorer_and_predict_on_two_gpus(tmp_path):
    _need_two_gpus()
    import torch.multiprocessing as mp
    mp.spawn(_scorer_worker, args=(2, 36500 + os.getpid() % 2000, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert np.load(os.path.join(str(tmp_path), "scorer_%d.npy" % r)).all()


def _calib_worker(rank, world, port, out_dir):
    torch, dist = _init(rank, world, port)
    from deepbind_b200 import cfg, hypertrain
    rng = np.random.default_rng(0)
    motif = "TGACGTCA"
    seqs, Y = [], []
    for i in range(600):
        s = "".join(rng.choice(list("ACGT"), size=40))
        if i % 2:
            p = int(rng.integers(0, 32)); s = s[:p] + motif + s[p + 8:]
        seqs.append(s); Y.append(float(i % 2))
    layers = cfg.loads("return [motif_scan(num_motifs=16, motif_len=12, init_scale=loguniform(1e-3, 1e-1)), bias(), rectify(), maxpool(),"
                       " full(num_units=1, init_scale=loguniform(1e-3, 1e-1)), bias(), softmax()]")
    spec = cfg.sgd(rate=cfg.loguniform(1e-3, 1e-1), momentum=0.9, batchsize=64, max_steps=120, checkpoints=2)
    recs, best = hypertrain.calibrate(layers, spec, seqs, Y, ncalib=5, nfold=2, seed=3, group="world")
    net, bt, vals = hypertrain.train_final(layers, spec, best, seqs, Y, ntrial=3, seed=3, group="world")
    params = hypertrain.best_trial_params(net, bt, 3, group="world")
    out = {"values": [r["value"] for r in recs], "keys": [(r["sample"], r["step"]) for r in recs], "best": (best["sample"], best["step"]),
           "vals": vals.tolist(), "bt": bt, "psum": float(sum(float(np.abs(v).sum()) for v in params.values()))}
    if rank == 0:                                            # the same search in one process, no group
        recs1, best1 = hypertrain.calibrate(layers, spec, seqs, Y, ncalib=5, nfold=2, seed=3)
        out["values1"] = [r["value"] for r in recs1]
        out["best1"] = (best1["sample"], best1["step"])
    np.save(os.path.join(out_dir, "calib_%d.npy" % rank), np.array([out], dtype=object), allow_pickle=True)
    dist.barrier()
    dist.destroy_process_group()


def test_calibration_dealt_to_two_gpus(tmp_path):
    _need_two_gpus()
    import torch.multiprocessing as mp
    mp.spawn(_calib_worker, args=(2, 38500 + os.getpid() % 2000, str(tmp_path)), nprocs=2, join=True)
    o = [np.load(os.path.join(str(tmp_path), "calib_%d.npy" % r), allow_pickle=True)[0] for r in range(2)]
    assert o[0]["keys"] == o[1]["keys"] and len(o[0]["keys"]) == 5 * 2
    assert o[0]["values"] == o[1]["values"] and o[0]["best"] == o[1]["best"]          # every rank holds every record
    assert o[0]["vals"] == o[1]["vals"] and o[0]["bt"] == o[1]["bt"] and o[0]["psum"] == o[1]["psum"]
    # an instance trains the same whichever GPU it lands on (up to the summation order of the launch shapes)
    np.testing.assert_allclose(o[0]["values"], o[0]["values1"], atol=2e-3)
    assert max(o[0]["values"]) > 0.9
