"""Committed golden fixtures (tests/golden/*.npz, written by make_golden.py).

On CPU the oracle must reproduce them exactly (it cannot drift unnoticed); on
the GPU the CUDA path is compared with the same committed numbers."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SCORING = ["pbm_forward", "genome_scan", "ragged_rna"]
TRAINING = ["chip_train", "calibration"]


def load(name):
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    params = {k[2:]: z[k] for k in z.files if k.startswith("p_")}
    return z, params


@pytest.mark.parametrize("name", SCORING)
def test_oracle_reproduces_scoring_fixture(orc, name):
    z, params = load(name)
    pool, I = str(z["pool"]), int(z["nmodel"])
    pooled, amax = orc.scanpool(params["Wscan"], params["bscan"], True, z["X"], z["R"], pool, True)
    assert np.array_equal(pooled, z["pooled"]) and np.array_equal(amax, z["argmax"])
    scores = orc.score_net(params, z["X"], z["R"], pool, I, strand_max=bool(z["strand_max"]))
    np.testing.assert_allclose(scores, z["scores"], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("name", TRAINING)
def test_oracle_reproduces_training_fixture(orc, name):
    z, params = load(name)
    mask = z["mask"] if z["mask"].size else None
    L, g = orc.train_grads(params, z["X"], z["R"], z["Y"], str(z["pool"]), int(z["nmodel"]), str(z["loss"]), mask)
    np.testing.assert_allclose(L, z["loss0"], rtol=1e-6)
    for k in g:
        np.testing.assert_allclose(g[k], z["g_" + k], rtol=1e-5, atol=1e-8)


def dev(a):
    import torch
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("name", SCORING)
def test_gpu_scoring_matches_fixture(cuda, name):
    from deepbind_b200 import fused
    from deepbind_b200.model import DeepBindNet
    z, params = load(name)
    pool, I = str(z["pool"]), int(z["nmodel"])
    X, R = dev(z["X"]), dev(z["R"])
    pooled, amax, _ = fused.scanpool(dev(params["Wscan"]), dev(params["bscan"]), X, R, pool, want_argmax=True)
    assert np.array_equal(pooled.cpu().numpy(), z["pooled"])                     # bit-exact
    assert np.array_equal(amax.cpu().numpy().view(np.uint32), z["argmax"])       # bit-exact
    net = DeepBindNet(params, I, pool)
    scores = net.score(X, R, strand_max=bool(z["strand_max"])).cpu().numpy()
    # dense head: summation order differs from the oracle's; fp32 tolerance 1e-5
    np.testing.assert_allclose(scores, z["scores"], rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("name", TRAINING)
def test_gpu_training_matches_fixture(cuda, name):
    from deepbind_b200.model import DeepBindNet
    z, params = load(name)
    pool, I = str(z["pool"]), int(z["nmodel"])
    X, R, Y = dev(z["X"]), dev(z["R"]), dev(z["Y"])
    mask = dev(z["mask"]) if z["mask"].size else None
    net = DeepBindNet(params, I, pool, loss=str(z["loss"]))
    L = net.grads(X, R, Y, mask).cpu().numpy()
    np.testing.assert_allclose(L, z["loss0"], rtol=1e-5)
    g = net.params_numpy("dP")
    for k in g:
        want = z["g_" + k]
        assert np.max(np.abs(g[k].reshape(want.shape) - want)) <= 1e-5 * max(np.abs(want).max(), 1e-6), k
    net.set_rates(z["rate"], float(z["momentum"]))
    for _ in range(int(z["nstep"])):
        net.train_step(X, R, Y, mask)
    P = net.P.cpu().numpy()
    assert np.max(np.abs(P - z["P_final"])) <= 1e-5 * np.abs(z["P_final"]).max()
    assert np.max(np.abs(net.mP.cpu().numpy() - z["mP_final"])) <= 1e-5 * max(np.abs(z["mP_final"]).max(), 1e-6)


def _predict_fixture():
    z, params = load("scan_predict")
    off = z["offsets"]
    text = z["text"].tobytes().decode("latin-1")
    seqs = [text[off[i]:off[i + 1]] for i in range(len(off) - 1)]
    return z, params, seqs


def test_oracle_reproduces_predict_fixture(orc):
    z, params, seqs = _predict_fixture()
    out = orc.predict(params, seqs, int(z["m"]), str(z["pool"]), int(z["nmodel"]), scan=int(z["scan"]), stride=int(z["stride"]),
                      reverse_complement=bool(z["reverse_complement"]))
    for k in ("direct", "max", "avg", "sum"):
        np.testing.assert_allclose(out[k], z[k], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(out["pmaps"][0], z["pmap0"], rtol=1e-6, atol=1e-7)


@pytest.mark.gpu
def test_gpu_predict_matches_fixture(cuda):
    from deepbind_b200.model import DeepBindNet
    from deepbind_b200.predict import predict
    z, params, seqs = _predict_fixture()
    net = DeepBindNet(params, int(z["nmodel"]), str(z["pool"]))
    got = predict(net, seqs, scan=int(z["scan"]), stride=int(z["stride"]), reverse_complement=bool(z["reverse_complement"]),
                  want_pmaps=True)
    for k in ("direct", "max", "avg", "sum"):
        np.testing.assert_allclose(got[k].cpu().numpy(), z[k], rtol=1e-5, atol=1e-5 if k == "sum" else 1e-6)
    np.testing.assert_allclose(got["pmaps"][0].cpu().numpy(), z["pmap0"], rtol=1e-5, atol=1e-6)
