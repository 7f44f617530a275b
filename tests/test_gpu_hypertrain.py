"""Calibration and final training end to end on a planted-motif toy problem."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ACGT = np.frombuffer(b"ACGT", dtype=np.uint8)

MODEL = """
return [motif_scan(num_motifs=16, motif_len=12, weight_decay=loguniform(1e-8,1e-5), init_scale=loguniform(1e-2,1e-1)),
        bias(), rectify(), maxpool(), dropout(rate=choice([0.0, 0.25])),
        full(num_units=1, weight_decay=loguniform(1e-8,1e-5), init_scale=loguniform(1e-2,1e-1)), bias(), softmax()]
"""


def planted(rng, n, L=40, motif="TGACGTCA"):
    seqs, y = [], []
    for i in range(n):
        s = ACGT[rng.integers(0, 4, L)].tobytes().decode()
        pos = i % 2
        if pos:
            at = int(rng.integers(0, L - len(motif)))
            s = s[:at] + motif + s[at + len(motif):]
        seqs.append(s); y.append(pos)
    return seqs, np.asarray(y, np.float32)


def test_calibrate_then_train(cuda, tmp_path):
    from deepbind_b200 import cfg
    from deepbind_b200.hypertrain import calibrate, train_final
    rng = np.random.default_rng(3)
    seqs, y = planted(rng, 600)
    layers = cfg.loads(MODEL)
    spec = cfg.sgd(rate=cfg.loguniform(0.01, 0.1), momentum=0.9, batchsize=50, max_epochs=100, max_steps=120, checkpoints=2,
                   weight_decay_start=20)
    records, best = calibrate(layers, spec, seqs, y, ncalib=4, nfold=3, seed=5, outdir=str(tmp_path))
    assert len(records) == 4 * 2 and {r["step"] for r in records} == {60, 120}
    assert all(len(r["folds"]) == 3 and r["metric"] == "auc" for r in records)
    assert best is not None and best["value"] == max(r["value"] for r in records if not np.isnan(r["value"]))
    assert best["value"] > 0.6                                  # the planted motif is learnable in 120 steps
    saved = json.load(open(os.path.join(str(tmp_path), "calib.all.json")))
    assert saved["best"]["sample"] == best["sample"] and len(saved["records"]) == 8
    again, best2 = calibrate(layers, spec, seqs, y, ncalib=4, nfold=3, seed=5)
    assert [r["value"] for r in again] == [r["value"] for r in records]          # same seeds, same kernels: same numbers
    net, trial, vals = train_final(layers, spec, best, seqs, y, ntrial=3, seed=5)
    assert net.I == 3 and 0 <= trial < 3 and vals[trial] == np.nanmax(vals) and vals[trial] > 0.6


def test_saved_model_scores_like_the_trained_one(cuda, tmp_path):
    """save_model / load_model: all instances, and one instance cut out of a multi-instance net."""
    import torch
    from deepbind_b200 import cfg
    from deepbind_b200.hypertrain import load_model, save_model
    from deepbind_b200.predict import predict
    rng = np.random.default_rng(4)
    seqs, _ = planted(rng, 60)
    net, _ = cfg.instantiate(cfg.loads(MODEL), ninst=3, seed=7)
    want = predict(net, seqs)["direct"].cpu().numpy()
    path = os.path.join(str(tmp_path), "model.npz")
    save_model(path, net, meta={"sample": 2, "rate": [0.01]})
    net2, meta = load_model(path)
    assert meta == {"sample": 2, "rate": [0.01]} and net2.I == 3 and net2.pool == net.pool and net2.loss == net.loss
    assert torch.equal(net2.P, net.P)
    np.testing.assert_array_equal(predict(net2, seqs)["direct"].cpu().numpy(), want)
    save_model(path, net, instance=1)
    one, _ = load_model(path)
    assert one.I == 1
    np.testing.assert_allclose(predict(one, seqs)["direct"].cpu().numpy()[:, 0], want[:, 1], rtol=1e-6, atol=1e-7)
