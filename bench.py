#!/usr/bin/env python
"""Benchmark of the DeepBind hot path on B200.

Workload (``config.workload``): the many-model genome scan -- ``--nmodel``
independent DeepBind models (16 motifs x 24 taps each, max+mean pooling, linear
head) score ``--nseq`` 101-nt sequences per GPU into a [nseq, nmodel] matrix.
Synthetic, seeded inputs in the reference's batch layout.  One "step" is one
pass over the whole batch.  With several GPUs every rank scores its own
sequences (weak scaling) and the score shards are all-gathered with NCCL; the same
line also carries a strong-scaling leg (the 1,000,000 sequences of the named
configuration split over the GPUs).

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
    ap.add_argument("--variant", default="f16", choices=["f16x2", "bf16x3", "bf16x2", "f16", "bf16", "f32"],
                    help="arithmetic of the scan: one 16-bit piece per weight on tcgen05 (f16 = TF32-grade, bf16), several pieces "
                         "(f16x2, bf16x3 = fp32-grade), or the exact FP32 lookup-add kernel")
    ap.add_argument("--gather-chunks", type=int, default=16, help="pieces of the shard: upload, scan and read-back of the host-to-host call overlap piece by piece; "
                                                                       "with --gather nccl also the chunks whose all-gather overlaps the scan")
    ap.add_argument("--gather", choices=["peer", "nccl"], default="peer",
                    help="several GPUs: 'peer' = the scan kernel stores every score into all ranks' matrices over NVLink "
                         "(symmetric memory, no collective pass); 'nccl' = chunked all-gather overlapped with the scan")
    ap.add_argument("--nccl-max-ctas", type=int, default=8, help="several GPUs: CTAs NCCL may use per collective (0 = NCCL's default); "
                                                                  "the scan wants every SM")
    ap.add_argument("--no-variants", action="store_true", help="skip the short runs of the other arithmetic variants")
    ap.add_argument("--cpu-sample", type=int, default=8192, help="sequences in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the short runs of the other benchmark configurations")
    ap.add_argument("--calibration-models", type=int, default=90,
                    help="models of the calibration-sweep leg on one GPU (90 = the configuration; 12 = one rank's share on 8 GPUs)")
    ap.add_argument("--only-reference-kernels", action="store_true",
                    help="run only the comparison of the unfused operators with the reference's own kernels and print its JSON")
    return ap.parse_args()


def config(args, world):
    return {"workload": "many-model genome scan: %d models x %d motifs x %d taps, %d-nt uniform ACGT, max+avg pooling, "
                        "linear head, score matrix [nseq, %d]" % (args.nmodel, NMOTIF, M, L, args.nmodel),
            "nseq_per_gpu": args.nseq, "global_nseq": args.nseq * world, "nmodel": args.nmodel,
            "parallelism": "sequences sharded over %d GPU(s)%s" % (world, "" if world == 1 else
                                                                   ", scores stored by the scan kernel into every rank's matrix over NVLink (peer stores), one-element all-reduce as barrier"
                                                                   if args.gather == "peer" else
                                                                   ", NCCL all-gather of the score shards in %d chunks overlapped with the scan" % args.gather_chunks),
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
            "config": dict(config(args, world), variant=args.variant, tolerance_vs_fp32_reference=VARIANTS[args.variant][2]),
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "the reference has no CPU implementation of this path (CUDA-only); this arm times the CPU "
                    "restatement used as the parity oracle (float32, exact) on a sample of %d of the workload's sequences "
                    "per step: the cost per sequence does not depend on the batch size" % args.cpu_sample}
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
    "f16":    (1, "f16 (one f16 piece per prescaled weight on tcgen05: 11-bit weights, exact one-hot operand, fp32 accumulate; "
                  "<=5e-4 of the fp32 reference, inside the 2e-3 set for bf16/TF32 tensor-core paths)", 5e-4),
    "f16x2":  (2, "f16x2 (two f16 pieces per prescaled weight on tcgen05, fp32 accumulate; <=3e-6 of the fp32 reference)", 3e-6),
    "bf16x3": (3, "bf16x3 (three bf16 pieces per weight on tcgen05, fp32 accumulate; <=1e-5 of the fp32 reference)", 1e-5),
    "bf16x2": (2, "bf16x2 (two bf16 pieces per weight, fp32 accumulate; <=1e-5)", 1e-5),
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


PEAKS_FILE = os.environ.get("DEEPBIND_PEAKS_FILE", os.path.join(ROOT, "MEASURED_PEAKS.json"))


def _read_peaks():
    """Measured peaks of the GPU pool (copy bandwidth, cuBLAS bf16 burst and sustained); {} if the file is absent."""
    return json.load(open(PEAKS_FILE)) if os.path.exists(PEAKS_FILE) else {}


def side_workloads(dev, with_cpu, calibration_models=90):
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
    ms_exact = _events_ms(graph.replay, 50)
    # one launch instead of three: the tensor-core scan with two f16 pieces per weight and the linear head in its
    # epilogue (exact products, fp32 accumulation; the difference from the exact kernel's scores is measured here)
    exact = net.score(X, R)
    net.prepare_tc("f16x2")
    tc_scores = net.score_tc(X, R)
    tc_err = float((tc_scores - exact).abs().max() / exact.abs().max())
    tc_status = torch.zeros(1, dtype=torch.int32, device=dev)
    tc_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(tc_graph):
        net.score_tc(X, R, check=False, out=tc_scores, status=tc_status)
    for _ in range(3):
        tc_graph.replay()
    ms_tc = _events_ms(tc_graph.replay, 50)
    use_tc = tc_err <= 1e-5 and ms_tc < ms_exact and int(tc_status.item()) == 0
    ms = ms_tc if use_tc else ms_exact
    out["pbm_forward"] = {"unit": "sequences/s", "value": 4096 / ms * 1e3, "ms": ms, "ms_separate_launches": ms_eager,
                          "ms_exact_f32_kernel_graph": ms_exact, "ms_tensor_core_f16x2_graph": ms_tc,
                          "tensor_core_max_abs_err_over_max_abs_score": tc_err,
                          "kernel": "tcgen05 scan with the linear head in its epilogue, two f16 pieces per weight (<= 1e-5 of the exact "
                                    "kernel's scores, measured beside); one launch, replayed from a CUDA graph" if use_tc else
                                    "f32 lookup-add, bit-exact; scan + linear head replayed from a CUDA graph",
                          "cpu": cpu_time(lambda: orc.score_net(p, Xh, Rh, "max", 1), 4096),
                          "bound": "launch latency (99 M adds; one launch)" if use_tc else
                                   "launch latency (99 M adds; one scan launch + two head launches)",
                          **rates(int((Rh[:, 1] - Rh[:, 0]).sum()), NMOTIF, M, ms)}

    # config 5: ragged both-strand RNA scoring, 200000 x U{20..200} nt, 5 % N, 16 x 16 filters, strand max
    p = synth.model_params(1, 16, 51, "max")
    Xh, Rh = synth.ragged_batch(200000, 20, 200, 16, seed=52, n_frac=0.05, both_strands=True)
    net = DeepBindNet(p, 1, "max"); X, R = to_dev(Xh, Rh)
    for _ in range(3):
        net.score(X, R, strand_max=True)
    ms_exact = _events_ms(lambda: net.score(X, R, strand_max=True), 10)
    exact = net.score(X, R, strand_max=True)
    # the same scores from the tensor-core scan with two f16 pieces per weight (fp32-grade: the products are
    # exact, only the summation order differs); 16 filters fill an eighth of a 128-row tile
    net.prepare_tc("f16x2")
    tc_out = net.score_tc(X, R, strand_max=True)
    tc_err = float((tc_out - exact).abs().max() / exact.abs().max())
    for _ in range(3):
        net.score_tc(X, R, strand_max=True, check=False)
    ms_tc = _events_ms(lambda: net.score_tc(X, R, strand_max=True, check=False), 10)
    ms = min(ms_exact, ms_tc) if tc_err <= 1e-5 else ms_exact
    ns = 20000
    out["ragged_rna"] = {"unit": "sequences/s", "value": 200000 / ms * 1e3, "ms": ms,
                         "ms_exact_f32_kernel": ms_exact, "ms_tensor_core_f16x2": ms_tc,
                         "tensor_core_max_abs_err_over_max_abs_score": tc_err,
                         "kernel": ("tcgen05 scan, two f16 pieces per weight (<= 1e-5 of the exact kernel's scores, measured beside); "
                                    "strand maximum by db_strand_max") if (ms == ms_tc and ms_tc < ms_exact) else
                                   "f32 lookup-add, bit-exact; strand maximum by db_strand_max",
                         "cpu": cpu_time(lambda: orc.score_net(p, Xh[:Rh[2 * ns - 1, 1] + 15], Rh[:2 * ns], "max", 1, strand_max=True), ns),
                         "bound": "tensor pipe (8 MMAs of 128 x 256 x 16 per 256 rows; 16 of the tile's 128 filter rows are distinct)"
                         if (ms == ms_tc and ms_tc < ms_exact) else "shared-memory operand return path", "hbm_gbs_algorithmic": (Xh.size + 4 * 200000) / (ms * 1e-3) / 1e9,
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
        K = 32                                        # steps per replay: a replay costs the host about as much as two small steps take on the GPU
        graph, _ = net.capture_train_step(Xs, R1, Ys, Ms, feed=feed, steps=K)

        def step():
            graph.replay()
        for _ in range(200 // K):                     # replays are tens of microseconds: warm up past the clock ramp
            step()
        ms7 = _events_ms(step, reps // K) / K
        # the same steps as two launches each (db_ministep): a CTA per sample runs the whole chain, a second
        # kernel adds the samples' gradient shares and updates; the minibatch is read in place from the dataset
        net2 = DeepBindNet(p, I, pool, loss=loss)
        net2.set_rates(lr, 0.9)
        mstep = net2.ministep(Xall, R1, Yall, Mall, max_rows=L + M - 1)
        ms2 = None
        if mstep is not None:
            graph2 = mstep.capture(steps=K)
            for _ in range(200 // K):
                graph2.replay()
            ms2 = _events_ms(graph2.replay, reps // K) / K
            torch.cuda.synchronize()
            if int(mstep.status.item()) != 0 or not bool(torch.isfinite(net2.P).all()):
                ms2 = None                            # a failed or diverged run is not a timing
        ms = ms7 if ms2 is None else min(ms7, ms2)
        cpu = None
        if with_cpu:
            mk = (np.random.default_rng(1).random((B, npool * I)) >= 0.5) if hidden else None
            Xb = np.concatenate([Xh[:rows], np.full(M - 1, 255, np.uint8)])
            t = time.perf_counter()
            for _ in range(cpu_steps):
                orc.train_grads(p, Xb, Rh[:B], np.tile(Yh[0], (1, I)), pool, I, loss, mk)
            cpu = cpu_steps * B * I / (time.perf_counter() - t)
        out[name] = {"unit": "train samples/s (model x sample)", "value": I * B / ms * 1e3, "ms_per_step": ms,
                     "models": I, "minibatch": B,
                     "kernel": ("f32, two launches per step (sample-parallel chain + update), CUDA-graph replay (%d steps per replay)" % K)
                     if (ms2 is not None and ms2 <= ms7) else
                     ("f32 fused scan+pool forward/backward, seven launches per step, CUDA-graph replay (%d steps per replay)" % K),
                     "ms_per_step_seven_launches": ms7, "ms_per_step_two_launches": ms2,
                     "cpu": cpu, "adds_counted": "dense equivalent: forward scan + recompute + filter gradient = 3 scans of the minibatch "
                                                "(with max pooling alone the backward kernel visits only the argmax rows)",
                     **rates(B * (L + M - 1), NMOTIF * I, M, ms, passes=3)}

    # config 2: ChIP-seq-style training, one model, minibatch 128, allpool -> 32 hidden (dropout 0.5) -> sigmoid
    train("chip_train", 1, 128, 101, "all", 32, "nll", 64, 2000, 5)
    # config 3: calibration sweep, 90 independent models trained at once on 40-nt probes, minibatch 64
    train("calibration", calibration_models, 64, 40, "max", 0, "mse", 64, 1000, 1)
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
    K = 32                                            # steps per replay
    # few models per GPU: the two-launch step (a CTA per sample and model) where its gradient shares stay small
    mstep = net.ministep(Xall, R1, Yall, None, max_rows=Lc + M - 1)
    if mstep is not None and mstep.scratch_bytes <= (8 << 20):
        graph, loss = mstep.capture(steps=K), mstep.loss
        path = "two launches per step"
    else:
        graph, loss = net.capture_train_step(Xs, R1, Ys, None, feed=feed, steps=K)
        path = "seven launches per step"
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
            "models_per_gpu": [NMODEL // world, nmax], "minibatch": B, "losses_finite": finite, "step": path,
            "parallelism": "models dealt round robin to %d GPUs, no gradient exchange; all-gather of the loss vector" % world}


def reference_kernels(dev):
    """Device time of the reference's own kernels (compiled for sm_100a from the reference
    sources into the checker library, launched with the reference's geometry) beside the
    drop-in operators and the fused kernel on the same inputs: 16384 x 101 nt, 16 filters x
    24 taps, Z = 130 MB (larger than L2).  None when the checker library is not built."""
    import ctypes
    import torch
    so = os.path.join(ROOT, "oracle", "_ref", "libdeepbind_ref.so")
    if not os.path.exists(so):
        return None
    ref = ctypes.CDLL(so)
    from deepbind_b200 import fused, synth, smat as sm, kangaroo_smat as ks
    m, nf, nseq = 24, 16, 16384
    Xh, Rh = synth.uniform_batch(nseq, 101, m, seed=1)
    rng = np.random.default_rng(2)
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(np.float32)
    b = rng.uniform(-0.1, 0, nf).astype(np.float32)
    n = Xh.size - m + 1
    tX = torch.zeros(Xh.size + 256, dtype=torch.uint8, device=dev)      # the reference's loader reads whole words past the end
    tX[:Xh.size] = torch.from_numpy(Xh).to(dev)
    tX = tX[:Xh.size]
    tW, tb = torch.from_numpy(W).to(dev), torch.from_numpy(b).to(dev)
    tR = torch.from_numpy(Rh.view(np.int32)).to(dev)
    Z = torch.zeros((Xh.size, nf), dtype=torch.float32, device=dev)
    Pt = torch.empty((nseq, 2 * nf), dtype=torch.float32, device=dev)
    At = torch.empty((nseq, nf), dtype=torch.int32, device=dev)
    sW, sX, sR = sm.asarray(W), sm.asarray(Xh), sm.asarray(Rh)
    sZ = sm.sarray(Z, np.float32)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    F32, ALL = 9, 3

    def t_of(fn, reps=20):
        for _ in range(3):
            fn()
        return _events_ms(fn, reps)
    # the new operators are called through the C ABI with their outputs allocated beforehand, as the
    # reference's are: a Python wrapper that allocates per call costs more than these kernels take
    from deepbind_b200 import _lib
    from ctypes import byref
    dll = _lib.load()
    sm.bind_stream()
    popt = _lib.c_poolrgn_options_t(); popt.ptype = ALL
    copt = _lib.c_corr1ord_options_t(); copt.padmode = 0; copt.nchannel = 4
    sPt, sAt0 = sm.sarray(Pt, np.float32), sm.sarray(At, np.uint32)
    t = {}
    t["ref_corr1ord"] = t_of(lambda: ref.ref_corr1ord(F32, P(tW), m, nf, P(tX), n, P(Z)))
    t["new_corr1ord"] = t_of(lambda: dll.api_corr1ord(sW._ptr, sX._ptr, sZ._ptr, byref(copt)))
    t["ref_poolrgn_all"] = t_of(lambda: ref.ref_poolrgn(F32, P(Z), nf, P(tR), nseq, 2, P(Pt), P(At), ALL))
    t["new_poolrgn_all"] = t_of(lambda: dll.api_poolrgn(sZ._ptr, sR._ptr, sPt._ptr, sAt0._ptr, byref(popt)))
    t["new_fused_scan_bias_relu_pool"] = t_of(lambda: fused.scanpool(tW, tb, sX.tensor.view(-1), tR, "all", want_argmax=True))
    dZ = torch.randn((Xh.size, nf), dtype=torch.float32, device=dev)
    dW = torch.zeros((4 * m, nf), dtype=torch.float32, device=dev)
    sdZ, sdW = sm.sarray(dZ, np.float32), sm.sarray(dW, np.float32)
    t["ref_corr1ord_bprop_W"] = t_of(lambda: ref.ref_corr1ord_bprop_W(F32, P(dW), m, nf, P(tX), n, P(dZ)))
    t["new_corr1ord_bprop_W"] = t_of(lambda: dll.api_corr1ord_bprop_W(sdW._ptr, sX._ptr, sdZ._ptr, byref(copt)))
    dP = torch.randn((nseq, 2 * nf), dtype=torch.float32, device=dev)
    sdP, sAt = sm.sarray(dP, np.float32), sm.sarray(At, np.uint32)
    ref.ref_poolrgn(F32, P(Z), nf, P(tR), nseq, 2, P(Pt), P(At), ALL)
    t["ref_poolrgn_bprop_all"] = t_of(lambda: ref.ref_poolrgn_bprop(F32, P(dZ), nf, P(tR), nseq, 2, P(dP), P(At), ALL))
    t["new_poolrgn_bprop_all"] = t_of(lambda: dll.api_poolrgn_bprop(sdZ._ptr, sR._ptr, sdP._ptr, sAt._ptr, byref(popt)))
    dXs = sm.zeros((Xh.size, 4), np.float32)
    t["new_corr1ord_bprop_X"] = t_of(lambda: dll.api_corr1ord_bprop_X(dXs._ptr, sW._ptr, sdZ._ptr, byref(copt)), reps=5)
    zbytes = float(Xh.size) * nf * 4
    peaks = _read_peaks()
    hbm = (peaks.get("hbm_gbs") or 6650.0) * 1e9
    out = {"unit": "ms per call", "case": "16384 x 101 nt, 16 filters x 24 taps; Z [npos, 16] f32 = %.0f MB" % (zbytes / 1e6),
           "ms": t, "z_bytes": zbytes,
           "scan_pool_chain_speedup": (t["ref_corr1ord"] + t["ref_poolrgn_all"]) / t["new_fused_scan_bias_relu_pool"],
           "frac_hbm": {"new_poolrgn_all": zbytes / (t["new_poolrgn_all"] * 1e-3) / hbm,
                        "new_poolrgn_bprop_all": 2 * zbytes / (t["new_poolrgn_bprop_all"] * 1e-3) / hbm,
                        "new_corr1ord": zbytes / (t["new_corr1ord"] * 1e-3) / hbm},
           "note": "reference kernels recompiled for sm_100a with their own launch geometry; frac_hbm = npos*nf*4 bytes per pass (read and written back by poolrgn_bprop, which adds into Z: twice that) "
                   "over the measured copy bandwidth (%s)" % ("measured" if "hbm_gbs" in peaks else "fallback 6650 GB/s")}
    return out


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist
    from deepbind_b200 import _lib, fused, shard, synth
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import ShardedScorer

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer stores only
        opts = None
        if args.nccl_max_ctas > 0:
            # The scan keeps one CTA on every SM (all of the SM's tensor memory); NCCL's copy CTAs take
            # SMs away from it while a chunk is gathered, so they are held to a few.
            try:
                opts = dist.ProcessGroupNCCL.Options()
                opts.config.max_ctas = args.nccl_max_ctas
                opts.config.min_ctas = min(args.nccl_max_ctas, 4)
            except (AttributeError, TypeError):
                opts = None
        dist.init_process_group("nccl", device_id=dev, **({"pg_options": opts} if opts is not None else {}))
    dll = _lib.load()
    if args.only_reference_kernels:
        print(json.dumps({"reference_kernels": reference_kernels(dev)}))
        return

    I, nseq = args.nmodel, args.nseq
    nsplit, dtype_name, tol = VARIANTS[args.variant]
    params = synth.model_params(I, M, 7, "all")
    net = DeepBindNet(params, I, "all")
    Xh, Rh = synth.uniform_batch(nseq, L, M, seed=1000 + rank)
    X_host = torch.from_numpy(Xh).pin_memory()
    R_host = torch.from_numpy(Rh.view(np.int32)).pin_memory()
    out_host = torch.empty((nseq, I), dtype=torch.float32).pin_memory()
    X = X_host.to(dev); R = R_host.to(dev)
    if nsplit:
        net.prepare_tc(args.variant)
    # nchunk: pieces of the host-to-host pipeline (upload, scan, read-back overlapped) and of the NCCL gather
    scorer = ShardedScorer(net, nseq, group=None, nchunk=args.gather_chunks, gather=args.gather)
    scores = scorer.scores
    status = scorer.status
    gathered = scorer.gathered

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if nsplit:
            scorer.run(X, R)                 # several GPUs: every chunk's all-gather overlaps the scan of the next
            return
        net.score_chunked(X, R, scores, args.chunk)
        if world > 1:
            dist.all_gather_into_tensor(gathered, scores)

    # The host-to-host call streams: it returns once a batch is enqueued, and the next batch's uploads and
    # scans overlap the last read-backs of this one (piece by piece dependencies); the timed region ends
    # when the last batch's scores are in host memory.
    stream_e2e = bool(nsplit) and (world == 1 or args.gather == "peer")

    def e2e_step():
        if nsplit:
            scorer.run_host(X_host, R_host, out_host, dev_bufs=(X, R, scores), wait=not stream_e2e)
            return
        net.predict_host(X_host, R_host, out_host, args.chunk, dev_bufs=(X, R, scores), tc=False)
        if world > 1:
            dist.all_gather_into_tensor(gathered, scores)

    def timed(fn, nstep, finish=None):
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(nstep):
            fn()
        if finish is not None:
            finish()                                  # everything enqueued has reached the host
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
    if nsplit:
        scorer.check()
    # outside the timed region: every rank's rows of the gathered matrix are its own scores, and all ranks
    # hold the same matrix
    gather_verified = scorer.verify() if (world > 1 and nsplit) else None
    e2e_step()
    if stream_e2e:
        scorer.wait_host()
    ms_e2e = timed(e2e_step, args.steps, finish=scorer.wait_host if stream_e2e else None)
    if nsplit:
        scorer.check()
    e2e_matches = None
    if nsplit:
        e2e_matches = bool(torch.equal(out_host[:4096], scores[:4096].cpu()))

    # dominant kernel alone: CUDA events on the launch stream around the scan launches of one step
    peaks = _read_peaks()
    prop = torch.cuda.get_device_properties(dev)
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 3)
    alg_bytes = nseq * ((L + M - 1) + I * 4)

    def tc_kernel_ms(reps):
        k0.record()
        for _ in range(reps):
            net.score_tc(X, R, check=False, out=scores, status=status)
        k1.record(); k1.synchronize()
        return k0.elapsed_time(k1) / reps
    dense_flop = 2.0 * 4 * M * (L + M - 1) * NMOTIF * I * nseq              # 2*K*rows*filters
    peak = peaks.get("bf16_tflops_sustained") or 1400.0
    src = "measured: cuBLAS bf16 GEMM run back to back under the power cap (sustained)" \
        if "bf16_tflops_sustained" in peaks else "fallback 1.4 PFLOP/s sustained"
    if nsplit:
        kernel_ms = tc_kernel_ms(reps)
        alg = dense_flop / (kernel_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "scanpool_tc_kernel (tcgen05 kind::f16, %s: %d piece(s) per weight)" % (args.variant, nsplit),
                    "achieved": alg, "peak": peak, "unit": "TFLOP/s", "frac": alg / peak, "peak_source": src,
                    "flops_counted": "algorithmic: dense-equivalent 2*K*rows*filters per sequence (K=96, 124 rows, 8192 filters at "
                                     "512 models); frac_executed counts every 16-bit piece of a weight the tensor cores multiply",
                    "frac_executed": nsplit * alg / peak, "executed_tflops": nsplit * alg,
                    "burst_peak": peaks.get("bf16_tflops"), "frac_of_burst": alg / peaks["bf16_tflops"] if peaks.get("bf16_tflops") else None,
                    "traffic": None,
                    "traffic_unit": "bytes per launch; algorithmic: %d.  One single-pass ncu capture of this launch (dram bytes read + "
                                    "written) gave 1.05 x the algorithmic bytes: the summary of the kernel's profile records it" % alg_bytes,
                    "ms_per_launch": kernel_ms, "hbm_gbs_algorithmic": alg_bytes / (kernel_ms * 1e-3) / 1e9}
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
        issue_peak = prop.multi_processor_count * 128 * sm_max * 1e6
        roofline = {"bound": "fp32-add-issue", "kernel": "scanpool_fwd_kernel<24> (FP32 lookup-add)",
                    "achieved": adds / (kernel_ms * 1e-3) / 1e12, "peak": issue_peak / 1e12, "unit": "Tadd/s",
                    "frac": adds / (kernel_ms * 1e-3) / issue_peak,
                    "frac_smem_operand_ceiling": adds / (kernel_ms * 1e-3) / (issue_peak / 4),
                    "peak_source": "SMs x 128 lanes x max SM clock (one FP32 add per lane and clock); the kernel fetches one 4-byte table "
                                   "operand per add from shared memory, whose return path allows a quarter of that",
                    "traffic": None, "ms_per_launch": kernel_ms}

    # the other arithmetic variants of the same workload, device-resident, a few launches each
    variants = None
    if world == 1 and nsplit and not args.no_variants:
        variants = {args.variant: {"value": nseq / (kernel_ms * 1e-3), "unit": UNIT, "tolerance_vs_fp32_reference": tol,
                                   "frac_algorithmic": roofline["frac"], "frac_executed": roofline["frac_executed"]}}
        for name in ("f16x2", "bf16", "f16", "bf16x3"):
            if name in variants:
                continue
            ns, _, vtol = VARIANTS[name]
            net.prepare_tc(name)
            for _ in range(2):
                net.score_tc(X, R, check=False, out=scores, status=status)
            vms = tc_kernel_ms(2)
            valg = dense_flop / (vms * 1e-3) / 1e12
            variants[name] = {"value": nseq / (vms * 1e-3), "unit": UNIT, "tolerance_vs_fp32_reference": vtol,
                              "frac_algorithmic": valg / peak, "frac_executed": ns * valg / peak}
        net.prepare_tc(args.variant)
        nsmall = min(nseq, 65536)                                # the exact FP32 kernel on a slice of the same batch
        f32_out = torch.empty((nsmall, I), dtype=torch.float32, device=dev)
        net.score_chunked(X, R[:nsmall], f32_out, args.chunk)
        fms = _events_ms(lambda: net.score_chunked(X, R[:nsmall], f32_out, args.chunk), 1)
        variants["f32"] = {"value": nsmall / (fms * 1e-3), "unit": UNIT, "tolerance_vs_fp32_reference": 0.0,
                           "sample": "%d of the batch's sequences" % nsmall,
                           "Tadd_per_s": adds_per_seq(I) * nsmall / (fms * 1e-3) / 1e12}
        # the scores of the headline variant against the exact kernel's on the same rows
        net.score_tc(X, R[:nsmall], check=True, out=scores[:nsmall])
        variants[args.variant]["max_abs_err_vs_f32_over_max_abs_score"] = \
            float((scores[:nsmall] - f32_out).abs().max() / f32_out.abs().max())
        del f32_out

    # strong scaling: the named configuration's 1,000,000 sequences split over the GPUs, gathered on every rank
    strong = None
    if world > 1 and nsplit:
        gn = 1000000
        lo, hi = shard.shard_range(gn, rank, world)
        n_s = gn // world                                        # equal shards (the remainder, < world sequences, is left out)
        sc = ShardedScorer(net, n_s, group=None, nchunk=max(1, min(args.gather_chunks, n_s // 8192)), gather=args.gather)
        Xs, Rs = X, R[:n_s]
        for _ in range(3):
            sc.run(Xs, Rs)
        ms_s = timed(lambda: sc.run(Xs, Rs), args.steps)
        sc.check()
        strong = {"global_nseq": n_s * world, "nseq_per_gpu": n_s, "value": n_s * world * args.steps / (ms_s * 1e-3), "unit": UNIT,
                  "ms_per_step": ms_s / args.steps, "gather_verified": sc.verify(), "gather": sc.gather, "chunks": sc.nchunk,
                  "note": "strong scaling: total work fixed at the configuration's 1,000,000 sequences; every rank ends with all scores"}
        del sc

    calib = calibration_sharded(dev, rank, world) if (world > 1 and not args.no_side) else None
    if rank == 0:
        line = {"metric": METRIC, "value": nseq * world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
                "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
                "config": dict(config(args, world), variant=args.variant, tolerance_vs_fp32_reference=tol),
                "clocks": clocks,
                "e2e": {"value": nseq * world * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                        "h2d_bytes_per_step": int(X_host.numel() + R_host.numel() * 4),
                        "d2h_bytes_per_step": int(out_host.numel() * 4), "ms_per_step": ms_e2e / args.steps,
                        "host_scores_match_device": e2e_matches,
                        "streamed": stream_e2e,
                        "note": "every step uploads its batch from pinned host memory and reads its scores back into pinned host "
                                "memory inside the timed region; with streamed = true a step's call returns once it is enqueued and the "
                                "next step's uploads and scans overlap its last read-backs, the region ending when the last step's scores "
                                "are in host memory"},
                "gpu_launches": launches, "roofline": roofline}
        if gather_verified is not None:
            line["gather_verified"] = gather_verified
        if variants is not None:
            line["variants"] = variants
        if strong is not None:
            line["strong_scaling"] = strong
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_run(args, args.cpu_sample, 1, 1)
        if world == 1 and not args.no_side:
            del X, R, scores, X_host, R_host, out_host, scorer
            torch.cuda.empty_cache()
            line["other_configs"] = side_workloads(dev, not args.no_cpu_baseline, args.calibration_models)
            rk = reference_kernels(dev)
            if rk is not None:
                line["other_configs"]["reference_kernels"] = rk
        if calib is not None:
            line["other_configs"] = {"calibration": calib}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
