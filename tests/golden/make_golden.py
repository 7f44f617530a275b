"""Writes the golden fixtures in this directory.

The reference cannot run here (Python 2, CUDA-only), so the fixtures are
produced by the CPU oracle, which is itself pinned by the known-answer tests in
tests/test_oracle_kat.py.  They freeze inputs and expected outputs of small
instances of the five benchmark configurations so that (a) the oracle cannot
drift unnoticed and (b) the GPU tests compare against committed numbers.

    python tests/golden/make_golden.py [case ...]
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as orc          # noqa: E402
from deepbind_b200 import synth           # noqa: E402


def flat(prefix, d):
    return {prefix + k: v for k, v in d.items()}


def scoring_case(name, X, R, params, pool, I, strand_max=False):
    pooled, amax = orc.scanpool(params["Wscan"], params["bscan"], True, X, R, pool, True)
    scores = orc.score_net(params, X, R, pool, I, strand_max=strand_max)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), X=X, R=R, pooled=pooled, argmax=amax, scores=scores,
                        pool=pool, nmodel=I, strand_max=strand_max, **flat("p_", params))


def training_case(name, X, R, params, pool, I, loss, Y, mask, rate, momentum, nstep):
    L, g = orc.train_grads(params, X, R, Y, pool, I, loss, mask)
    # a few Nesterov steps on the same minibatch
    P = orc.flatten(params).copy()
    mom = np.zeros_like(P)
    drate = np.concatenate([np.repeat(rate, params[k].size // I) if k in ("W1", "W2") else
                            np.tile(np.repeat(rate, params[k].shape[-1] // I), params[k].size // params[k].shape[-1])
                            for k in orc.PARAM_ORDER if k in params]).astype(np.float32)
    mrate = np.full_like(drate, momentum)
    losses = []

    def grad_fn(Pvec):
        Lk, gk = orc.train_grads(orc.unflatten(Pvec, params), X, R, Y, pool, I, loss, mask)
        losses.append(Lk)
        return orc.flatten(gk)

    for _ in range(nstep):
        orc.nesterov_step(P, mom, drate, mrate, grad_fn)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), X=X, R=R, Y=Y, mask=mask if mask is not None else np.zeros((0, 0), bool), loss0=L, rate=rate,
                        momentum=momentum, nstep=nstep, P_final=P, mP_final=mom, losses=np.array(losses),
                        pool=pool, nmodel=I, loss=loss, **flat("p_", params), **flat("g_", g))


def predict_case(name, seqs, params, m, pool, I, scan, stride, rc):
    """Direct and scan-mode predictions (kangaroo.predict semantics) of sequence strings."""
    out = orc.predict(params, seqs, m, pool, I, scan=scan, stride=stride, reverse_complement=rc)
    text = np.frombuffer("".join(seqs).encode("latin-1"), np.uint8)
    offsets = np.concatenate([[0], np.cumsum([len(s) for s in seqs])]).astype(np.int64)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), text=text, offsets=offsets, m=m, pool=pool, nmodel=I, scan=scan,
                        stride=stride, reverse_complement=rc, direct=out["direct"], max=out["max"], avg=out["avg"],
                        sum=out["sum"], pmap0=out["pmaps"][0], **flat("p_", params))


def case_pbm_forward():
    # 1. PBM-style forward scoring: 40-nt probes, 16 x 24 filters, maxpool, linear head
    X, R = synth.uniform_batch(64, 40, 24, seed=101)
    scoring_case("pbm_forward", X, R, synth.model_params(1, 24, 102, "max"), "max", 1)


def case_genome_scan():
    # 4. many-model scan: 6 models, 101-nt, allpool, linear head
    X, R = synth.uniform_batch(48, 101, 24, seed=401)
    scoring_case("genome_scan", X, R, synth.model_params(6, 24, 402, "all"), "all", 6)


def case_ragged_rna():
    # 5. ragged both-strand scoring with N, 16 x 16 filters, maxpool, strand max
    X, R = synth.ragged_batch(40, 20, 200, 16, seed=501, n_frac=0.05, both_strands=True)
    scoring_case("ragged_rna", X, R, synth.model_params(1, 16, 502, "max"), "max", 1, strand_max=True)


def case_chip_train():
    # 2. ChIP-style training: 101-nt, allpool -> 32 hidden -> sigmoid, dropout 0.5, nll
    g = synth.rng(201)
    X, R = synth.uniform_batch(32, 101, 24, seed=202)
    Y = g.integers(0, 2, size=(32, 1)).astype(np.float32)
    mask = g.random((32, 32)) >= 0.5
    training_case("chip_train", X, R, synth.model_params(1, 24, 203, "all", hidden=32), "all", 1, "nll", Y, mask,
                  np.array([0.01], np.float32), 0.9, 3)


def case_calibration():
    # 3. calibration: 5 models with different learning rates, 40-nt, maxpool, mse
    g = synth.rng(301)
    X, R = synth.uniform_batch(64, 40, 24, seed=302)
    Y = np.tile(g.standard_normal((64, 1)).astype(np.float32), (1, 5))
    rate = np.exp(g.uniform(np.log(1e-4), np.log(1e-1), 5)).astype(np.float32)
    training_case("calibration", X, R, synth.model_params(5, 24, 303, "max"), "max", 5, "mse", Y, None, rate, 0.9, 3)


def case_scan_predict():
    # predict driver: ragged sequences with N, 3 models, both strands, windows of 20 every 3 positions
    g = synth.rng(601)
    alphabet = np.frombuffer(b"ACGTN", np.uint8)
    seqs = [alphabet[g.choice(5, size=g.integers(8, 180), p=[.24, .24, .24, .24, .04])].tobytes().decode() for _ in range(24)]
    predict_case("scan_predict", seqs, synth.model_params(3, 16, 602, "max"), 16, "max", 3, 20, 3, True)


CASES = {f.__name__[5:]: f for f in (case_pbm_forward, case_genome_scan, case_ragged_rna, case_chip_train, case_calibration,
                                     case_scan_predict)}


if __name__ == "__main__":
    # python tests/golden/make_golden.py [case ...]   (no argument: every case)
    for name in (sys.argv[1:] or sorted(CASES)):
        CASES[name]()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))
