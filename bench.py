#!/usr/bin/env python
"""Benchmark of the DeepBind hot path on B200.

Workload (``config.workload``): the many-model genome scan -- ``--nmodel``
independent DeepBind models (16 motifs x 24 taps each, max+mean pooling, linear
head) score ``--nseq`` 101-nt sequences per GPU into a [nseq, nmodel] matrix.
Synthetic, seeded inputs in the reference's batch layout.  One "step" is one
pass over the whole batch.  With several GPUs every rank scores its own
sequences (weak scaling) and the score shards are all-gathered with NCCL.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # the CPU restatement, all host threads

Prints ONE JSON line (rank 0).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
# stdout carries one JSON line only: NCCL's version banner and warnings go to stderr (set before NCCL
# loads; NCCL honours the file only from level WARN up, and prints the banner at VERSION and WARN)
if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "WARN"
os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")

M, NMOTIF, L = 24, 16, 101
UNIT = "sequences/s"
METRIC = "sequences/sec scored"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--nseq", type=int, default=1000000, help="sequences per GPU")
    ap.add_argument("--nmodel", type=int, default=512)
    ap.add_argument("--chunk", type=int, default=16384, help="sequences per launch of the FP32 variant")
    ap.add_argument("--variant", default="f16x2", choices=["f16x2", "bf16x3", "bf16x2", "f16", "bf16", "f32"],
                    help="arithmetic of the scan: 16-bit weight pieces on tcgen05 (f16x2, bf16x3 = fp32-grade) or FP32 lookup-add")
    ap.add_argument("--gather-chunks", type=int, default=8, help="several GPUs: chunks of the shard whose all-gather overlaps the scan")
    ap.add_argument("--cpu-sample", type=int, default=8192, help="sequences in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the short runs of the other benchmark configurations")
    return ap.parse_args()


def config(args, world):
    return {"workload": "many-model genome scan: %d models x %d motifs x %d taps, %d-nt uniform ACGT, max+avg pooling, "
                        "linear head, score matrix [nseq, %d]" % (args.nmodel, NMOTIF, M, L, args.nmodel),
            "nseq_per_gpu": args.nseq, "global_nseq": args.nseq * world, "nmodel": args.nmodel,
            "parallelism": "sequences sharded over %d GPU(s), NCCL all-gather of score shards%s" % (world, " in %d chunks overlapped with the scan" % args.gather_chunks if world > 1 else ""),
            "l2": "working set per step (input + score matrix) exceeds the 126 MB L2; no explicit flush"}


def adds_per_seq(nmodel):
    return (L + M - 1) * NMOTIF * nmodel * M


# ------------------------------------------------------------------ CPU arm
def cpu_run(args, nsample, steps, warmup):
    """Times the CPU restatement of the path (the reference has no CPU code for it)
    with every host thread, on a bounded sample of the same workload."""
    from oracle import oracle as orc
    from deepbind_b200 import synth
    cores = len(os.sched_getaffinity(0))
    orc.set_num_threads(cores)
    params = synth.model_params(args.nmodel, M, 7, "all")
    X, R = synth.uniform_batch(nsample, L, M, seed=11)
    for _ in range(warmup):
        orc.score_net(params, X[:R[min(63, nsample - 1), 1] + M - 1], R[:64], "all", args.nmodel)
    times = []
    for _ in range(steps):
        t = time.perf_counter()
        orc.score_net(params, X, R, "all", args.nmodel)
        times.append(time.perf_counter() - t)
    dt = sum(times)
    # the same restatement on one thread, on a sixteenth of the sample
    n1 = max(64, nsample // 16)
    orc.set_num_threads(1)
    t = time.perf_counter()
    orc.score_net(params, X[:R[n1 - 1, 1] + M - 1], R[:n1], "all", args.nmodel)
    single = n1 / (time.perf_counter() - t)
    orc.set_num_threads(cores)
    return {"value": nsample * steps / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "%d of the workload's sequences x %d models per step, %d step(s), OpenMP over sequences"
                      % (nsample, args.nmodel, steps),
            "single_thread": {"value": single, "unit": UNIT, "sample": "%d sequences" % n1}}, dt / steps


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec = cpu_run(args, args.cpu_sample, max(1, args.steps), min(args.warmup, 1))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config(args, world), "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "the reference has no CPU implementation of this path (CUDA-only); this arm times the CPU "
                    "restatement used as the parity oracle"}
    print(json.dumps(line))


# ------------------------------------------------------------------ clocks
class ClockSampler(object):
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ GPU arm
VARIANTS = {
    # name: (16-bit pieces per weight, or None for the FP32 lookup-add kernel; dtype string; stated tolerance)
    "f16x2":  (2, "f16x2 (two f16 pieces per prescaled weight on tcgen05, fp32 accumulate; <=3e-6 of the fp32 reference)", 3e-6),
    "bf16x3": (3, "bf16x3 (three bf16 pieces per weight on tcgen05, fp32 accumulate; <=1e-5 of the fp32 reference)", 1e-5),
    "bf16x2": (2, "bf16x2 (two bf16 pieces per weight, fp32 accumulate; <=1e-5)", 1e-5),
    "f16":    (1, "f16 (prescaled weights, fp32 accumulate; <=5e-4)", 5e-4),
    "bf16":   (1, "bf16 (fp32 accumulate; <=2e-3)", 2e-3),
    "f32":    (None, "f32 (lookup-add, bit-exact pooling)", 0.0),
}


def _events_ms(fn, reps):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record(); e1.synchronize()
    return e0.elapsed_time(e1) / reps


def _read_peaks():
    """Peaks measured on this pool's GPUs (written beside this file by the harness); {} if absent."""
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    return json.load(open(pk)) if os.path.exists(pk) else {}


def side_workloads(dev, with_cpu):
    """Short device-timed runs of the other benchmark configurations (inputs resident
    in HBM, CUDA events, 3+ warm-up passes), each beside the CPU restatement timed on
    a bounded sample.  They ride along in the JSON line under `other_configs`."""
    import torch
    from deepbind_b200 import fused, synth
    from deepbind_b200.model import DeepBindNet
    from oracle import oracle as orc
    out = {}

    def to_dev(Xh, Rh):
        return torch.from_numpy(Xh).to(dev), torch.from_numpy(Rh.view(np.int32)).to(dev)

    def cpu_time(fn, units):
        if not with_cpu:
            return None
        t = time.perf_counter(); fn(); dt = time.perf_counter() - t
        return units / dt

    # FP32 add issue rate: SMs x 128 lanes x max SM clock, cross-checked by a register-only
    # chain of adds on every lane.  The lookup-add kernels fetch one table operand per add
    # from shared memory, whose return path (32 operands/clk/SM) is the tighter ceiling.
    from deepbind_b200 import _lib
    lib = _lib.load()
    prop = torch.cuda.get_device_properties(dev)
    sm_mhz = float(_read_peaks().get("sm_max_mhz") or 1965.0)
    issue_peak = prop.multi_processor_count * 128 * sm_mhz * 1e6
    for _ in range(3):
        lib.db_fadd_probe(None, 512)
    nadd = [0]

    def probe():
        nadd[0] = int(lib.db_fadd_probe(None, 4096))
    probe_ms = _events_ms(probe, 5)
    out["fp32_add_issue"] = {"unit": "Tadd/s", "nominal": issue_peak / 1e12, "measured_fadd_chain": nadd[0] / (probe_ms * 1e-3) / 1e12,
                             "smem_operand_ceiling": issue_peak / 4 / 1e12}

    def rates(rows, nf, m, ms, passes=1):
        """Lookup-adds of `passes` scans of `rows` buffer rows, against the two ceilings."""
        adds = float(rows) * nf * m * passes
        return {"adds": adds, "Tadd_per_s": adds / (ms * 1e-3) / 1e12, "frac_fp32_add_issue": adds / (ms * 1e-3) / issue_peak,
                "frac_smem_operand_ceiling": adds / (ms * 1e-3) / (issue_peak / 4)}

    # config 1: PBM-style forward scoring, 4096 x 40 nt, one model, exact FP32 kernel
    p = synth.model_params(1, M, 21, "max")
    Xh, Rh = synth.uniform_batch(4096, 40, M, seed=22)
    net = DeepBindNet(p, 1, "max"); X, R = to_dev(Xh, Rh)
    for _ in range(3):
        net.score(X, R)
    ms_eager = _events_ms(lambda: net.score(X, R), 20)
    graph, _ = net.capture_score(X, R)                       # the batch is launch-latency bound: replay it as one graph
    for _ in range(3):
        graph.replay()
    ms = _events_ms(graph.replay, 50)
    out["pbm_forward"] = {"unit": "sequences/s", "value": 4096 / ms * 1e3, "ms": ms, "ms_separate_launches": ms_eager,
                          "kernel": "f32 lookup-add, bit-exact; scan + linear head replayed from a CUDA graph",
                          "cpu": cpu_time(lambda: orc.score_net(p, Xh, Rh, "max", 1), 4096),
                          "bound": "launch latency (99 M adds; one scan launch + two head launches)",
                          **rates(int((Rh[:, 1] - Rh[:, 0]).sum()), NMOTIF, M, ms)}

    # config 5: ragged both-strand RNA scoring, 200000 x U{20..200} nt, 5 % N, 16 x 16 filters, strand max
    p = synth.model_params(1, 16, 51, "max")
    Xh, Rh = synth.ragged_batch(200000, 20, 200, 16, seed=52, n_frac=0.05, both_strands=True)
    net = DeepBindNet(p, 1, "max"); X, R = to_dev(Xh, Rh)
    for _ in range(3):
        net.score(X, R, strand_max=True)
    ms = _events_ms(lambda: net.score(X, R, strand_max=True), 10)
    ns = 20000
    out["ragged_rna"] = {"unit": "sequences/s", "value": 200000 / ms * 1e3, "ms": ms, "kernel": "f32 lookup-add, bit-exact",
                         "cpu": cpu_time(lambda: orc.score_net(p, Xh[:Rh[2 * ns - 1, 1] + 15], Rh[:2 * ns], "max", 1, strand_max=True), ns),
                         "bound": "shared-memory operand return path", "hbm_gbs_algorithmic": (Xh.size + 4 * 200000) / (ms * 1e-3) / 1e9,
                         **rates(int((Rh[:, 1] - Rh[:, 0]).sum()), NMOTIF, 16, ms)}
    del X, R

    def train(name, I, B, L, pool, hidden, loss, nbatch, reps, cpu_steps):
        """Minibatch steps (fetch of the next minibatch of the resident dataset, forward,
        backward, Nesterov update) replayed from a CUDA graph."""
        p = synth.model_params(I, M, 31, pool, hidden=hidden)
        g = synth.rng(32)
        Xh, Rh = synth.uniform_batch(B * nbatch, L, M, seed=33)
        rows = B * (L + M - 1)
        tail = M - 1 + (-(rows + M - 1)) % 16         # closing pad, grown so that a minibatch is whole 16-byte units
        Xall = torch.from_numpy(np.stack([np.concatenate([Xh[i * rows:(i + 1) * rows], np.full(tail, 255, np.uint8)])
                                          for i in range(nbatch)])).to(dev)
        R1 = torch.from_numpy(Rh[:B].view(np.int32)).to(dev)
        Yh = g.integers(0, 2, size=(nbatch, B, 1)).astype(np.float32) if loss == "nll" else \
            g.standard_normal((nbatch, B, 1)).astype(np.float32)
        Yall = torch.from_numpy(np.tile(Yh, (1, 1, I))).to(dev)
        npool = NMOTIF * (2 if pool == "all" else 1)
        Mall = torch.from_numpy(g.random((nbatch, B, npool * I)) >= 0.5).to(dev) if hidden else None
        net = DeepBindNet(p, I, pool, loss=loss)
        lr = np.exp(g.uniform(np.log(1e-4), np.log(1e-1), I)).astype(np.float32) if I > 1 else 0.01
        net.set_rates(lr, 0.9)
        Xs, Ys = Xall[0].clone(), Yall[0].clone()
        Ms = Mall[0].clone() if Mall is not None else None
        feed = fused.MinibatchFeed([(Xall, Xs), (Yall, Ys)] + ([(Mall, Ms)] if Ms is not None else []))
        K = 8                                         # steps per replay: the host's cost of a replay is above a small step's GPU time
        graph, _ = net.capture_train_step(Xs, R1, Ys, Ms, feed=feed, steps=K)

        def step():
            graph.replay()
        for _ in range(200 // K):                     # replays are tens of microseconds: warm up past the clock ramp
            step()
        ms = _events_ms(step, reps // K) / K
        cpu = None
        if with_cpu:
            mk = (np.random.default_rng(1).random((B, npool * I)) >= 0.5) if hidden else None
            Xb = np.concatenate([Xh[:rows], np.full(M - 1, 255, np.uint8)])
            t = time.perf_counter()
            for _ in range(cpu_steps):
                orc.train_grads(p, Xb, Rh[:B], np.tile(Yh[0], (1, I)), pool, I, loss, mk)
            cpu = cpu_steps * B * I / (time.perf_counter() - t)
        out[name] = {"unit": "train samples/s (model x sample)", "value": I * B / ms * 1e3, "ms_per_step": ms,
                     "models": I, "minibatch": B, "kernel": "f32 fused scan+pool forward/backward, CUDA-graph replay (%d steps per replay)" % K,
                     "cpu": cpu, "adds_counted": "dense equivalent: forward scan + recompute + filter gradient = 3 scans of the minibatch "
                                                "(with max pooling alone the backward kernel visits only the argmax rows)",
                     **rates(B * (L + M - 1), NMOTIF * I, M, ms, passes=3)}

    # config 2: ChIP-seq-style training, one model, minibatch 128, allpool -> 32 hidden (dropout 0.5) -> sigmoid
    train("chip_train", 1, 128, 101, "all", 32, "nll", 64, 2000, 5)
    # config 3: calibration sweep, 90 independent models trained at once on 40-nt probes, minibatch 64
    train("calibration", 90, 64, 40, "max", 0, "mse", 64, 1000, 1)
    return out


def calibration_sharded(dev, rank, world):
    """Config 3 over several GPUs: the 90 independent models of the calibration sweep are
    dealt to the ranks round robin (as hypertrain deals its samples to worker processes),
    every rank trains its own models on the same resident 40-nt data, CUDA-graph replay,
    and the only exchange is the all-gather of the per-model loss vector at the end.
    Time = CUDA events on every rank, maximum over ranks."""
    import torch
    import torch.distributed as dist
    from deepbind_b200 import fused, shard, synth
    from deepbind_b200.model import DeepBindNet
    NMODEL, B, Lc, nbatch, reps = 90, 64, 40, 64, 1000
    ids = shard.shard_models(NMODEL, rank, world)
    I = len(ids)
    g = synth.rng(32)
    p = synth.model_params(I, M, 31 + rank, "max")
    Xh, Rh = synth.uniform_batch(B * nbatch, Lc, M, seed=33)
    rows = B * (Lc + M - 1)
    tail = M - 1 + (-(rows + M - 1)) % 16             # closing pad, grown so that a minibatch is whole 16-byte units
    Xall = torch.from_numpy(np.stack([np.concatenate([Xh[i * rows:(i + 1) * rows], np.full(tail, 255, np.uint8)])
                                      for i in range(nbatch)])).to(dev)
    R1 = torch.from_numpy(Rh[:B].view(np.int32)).to(dev)
    Yall = torch.from_numpy(np.tile(g.standard_normal((nbatch, B, 1)).astype(np.float32), (1, 1, I))).to(dev)
    lr_all = np.exp(g.uniform(np.log(1e-4), np.log(1e-1), NMODEL)).astype(np.float32)
    net = DeepBindNet(p, I, "max", loss="mse")
    net.set_rates(lr_all[ids], 0.9)
    Xs, Ys = Xall[0].clone(), Yall[0].clone()
    feed = fused.MinibatchFeed([(Xall, Xs), (Yall, Ys)])
    K = 8                                             # steps per replay
    graph, loss = net.capture_train_step(Xs, R1, Ys, None, feed=feed, steps=K)
    nmax = (NMODEL + world - 1) // world
    mine = torch.zeros(nmax, dtype=torch.float32, device=dev)
    everyone = torch.empty(world * nmax, dtype=torch.float32, device=dev)

    def run(n):
        for _ in range(n // K):
            graph.replay()                            # K times: fetch of the next minibatch + training step
        mine[:I] = loss.view(-1)[:I]
        dist.all_gather_into_tensor(everyone, mine)
    run(200)
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); run(reps); e1.record()
    dist.barrier(); torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / reps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    finite = bool(torch.isfinite(everyone.view(world, nmax)[rank, :I]).all().item())
    return {"unit": "train samples/s (model x sample)", "value": NMODEL * B / ms * 1e3, "ms_per_step": ms, "models": NMODEL,
            "models_per_gpu": [NMODEL // world, nmax], "minibatch": B, "losses_finite": finite,
            "parallelism": "models dealt round robin to %d GPUs, no gradient exchange; all-gather of the loss vector" % world}


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist
    from deepbind_b200 import _lib, fused, shard, synth
    from deepbind_b200.model import DeepBindNet

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dll = _lib.load()

    I, nseq = args.nmodel, args.nseq
    nsplit, dtype_name, tol = VARIANTS[args.variant]
    params = synth.model_params(I, M, 7, "all")
    net = DeepBindNet(params, I, "all")
    Xh, Rh = synth.uniform_batch(nseq, L, M, seed=1000 + rank)
    X_host = torch.from_numpy(Xh).pin_memory()
    R_host = torch.from_numpy(Rh.view(np.int32)).pin_memory()
    out_host = torch.empty((nseq, I), dtype=torch.float32).pin_memory()
    X = X_host.to(dev); R = R_host.to(dev)
    scores = torch.empty((nseq, I), dtype=torch.float32, device=dev)
    gathered = torch.empty((nseq * world, I), dtype=torch.float32, device=dev) if world > 1 else None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    if nsplit:
        net.prepare_tc(args.variant)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def score():
        if nsplit:
            net.score_tc(X, R, check=False, out=scores, status=status)
        else:
            net.score_chunked(X, R, scores, args.chunk)

    # Several GPUs: the shard is scored in chunks and every chunk's all-gather (NCCL, its own
    # stream) runs while the next chunk is scored; `gathered_chunks` is chunk-major, rank-major
    # inside a chunk (shard.gathered_rows gives the flat order).
    gathered_chunks = None
    if world > 1 and nsplit:
        gathered_chunks = [gathered[world * lo:world * hi] for lo, hi in
                           (shard.shard_range(nseq, c, args.gather_chunks) for c in range(args.gather_chunks))]

    def score_rows(lo, hi):
        net.score_tc(X, R[lo:hi], check=False, out=scores[lo:hi], status=status)

    def step():
        if gathered_chunks is not None:
            shard.chunked_gather(score_rows, scores, gathered_chunks)
            return
        score()
        if world > 1:
            dist.all_gather_into_tensor(gathered, scores)

    def e2e_step():
        net.predict_host(X_host, R_host, out_host, args.chunk, dev_bufs=(X, R, scores), tc=bool(nsplit))
        if world > 1:
            dist.all_gather_into_tensor(gathered, scores)

    def timed(fn, nstep):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(nstep):
            fn()
        ev1.record()
        barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    l0 = dll.api_launch_count()
    ms = timed(step, args.steps)
    launches = int(dll.api_launch_count() - l0)
    clocks = sampler.stop() if sampler else None
    e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    if int(status.item()) != 0:
        raise SystemExit("tensor-core scan reported status %d" % int(status.item()))

    # dominant kernel alone: CUDA events on the launch stream around the scan launches of one step
    peaks = _read_peaks()
    prop = torch.cuda.get_device_properties(dev)
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 3)
    if nsplit:
        k0.record()
        for _ in range(reps):
            net.score_tc(X, R, check=False, out=scores, status=status)
        k1.record(); k1.synchronize()
        kernel_ms = k0.elapsed_time(k1) / reps
        dense_flop = 2.0 * 4 * M * (L + M - 1) * NMOTIF * I * nseq          # 2*K*rows*filters
        exec_flop = nsplit * dense_flop
        peak = peaks.get("bf16_tflops_sustained") or 1400.0
        src = "MEASURED_PEAKS.json bf16_tflops_sustained (cuBLAS bf16 GEMM run back to back under the power cap)" \
            if "bf16_tflops_sustained" in peaks else "fallback 1.4 PFLOP/s sustained"
        roofline = {"bound": "tensor", "kernel": "scanpool_tc_kernel (tcgen05 kind::f16, %s: %d piece(s) per weight)" % (args.variant, nsplit),
                    "achieved": exec_flop / (kernel_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                    "frac": exec_flop / (kernel_ms * 1e-3) / 1e12 / peak, "peak_source": src,
                    "flops_counted": "executed tensor flops = %d x dense-equivalent 2*K*rows*filters (K=96); the pieces are what "
                                     "fp32-grade results cost on 16-bit tensor cores (f16 and bf16 run at the same rate)" % nsplit,
                    "dense_equiv_tflops": dense_flop / (kernel_ms * 1e-3) / 1e12,
                    "burst_peak": peaks.get("bf16_tflops"),
                    # ncu, one launch of 1,000,000 sequences x 512 models: dram__bytes_read.sum 277 MB +
                    # dram__bytes_write.sum 2.01 GB (profiles/scanpool_tc_f16x2_genome_scan.md); it grows with the
                    # sequence count once the score matrix exceeds L2, so it is scaled from that capture
                    "traffic": (2.287e9 * nseq / 1e6) if (I == 512 and nseq >= 250000) else None,
                    "traffic_unit": "bytes per launch (algorithmic: %d)" % (nseq * ((L + M - 1) + I * 4)),
                    "ms_per_launch": kernel_ms,
                    "hbm_gbs_algorithmic": (nseq * ((L + M - 1) + I * 4)) / (kernel_ms * 1e-3) / 1e9}
    else:
        Wd, bd = net.view("Wscan"), net.view("bscan").view(-1)
        nchunk = (nseq + args.chunk - 1) // args.chunk
        ktime = 0.0
        for _ in range(min(reps, 2)):
            for s in range(0, nseq, args.chunk):
                Rc = R[s:min(nseq, s + args.chunk)]
                k0.record()
                fused.scanpool(Wd, bd, X, Rc, "all", relu=True)
                k1.record(); k1.synchronize()
                ktime += k0.elapsed_time(k1)
        kernel_ms = ktime / (min(reps, 2) * nchunk)
        adds = adds_per_seq(I) * nseq / nchunk                    # per launch, on average (the last chunk may be short)
        sm_max = (clocks or {}).get("sm_max_mhz") or peaks.get("sm_max_mhz") or 1965.0
        lut_peak = prop.multi_processor_count * 32 * sm_max * 1e6
        roofline = {"bound": "smem-lookup", "kernel": "scanpool_fwd_kernel<24> (FP32 lookup-add)",
                    "achieved": adds / (kernel_ms * 1e-3) / 1e12, "peak": lut_peak / 1e12, "unit": "Tadd/s",
                    "frac": adds / (kernel_ms * 1e-3) / lut_peak,
                    "peak_source": "SMs x 32 table operands/clk x max SM clock (shared-memory return path, one 4-byte operand "
                                   "per add); FP32 add issue would be 4x this", "traffic": None, "ms_per_launch": kernel_ms}

    calib = calibration_sharded(dev, rank, world) if (world > 1 and not args.no_side) else None
    if rank == 0:
        line = {"metric": METRIC, "value": nseq * world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
                "config": dict(config(args, world), variant=args.variant, tolerance_vs_fp32_reference=tol),
                "clocks": clocks,
                "e2e": {"value": nseq * world * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": int(X_host.numel() + R_host.numel() * 4),
                        "d2h_bytes_per_step": int(out_host.numel() * 4), "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": launches, "roofline": roofline}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_run(args, args.cpu_sample, 1, 1)
        if world == 1 and not args.no_side:
            del X, R, scores, X_host, R_host, out_host
            torch.cuda.empty_cache()
            line["other_configs"] = side_workloads(dev, not args.no_cpu_baseline)
        if calib is not None:
            line["other_configs"] = {"calibration": calib}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
