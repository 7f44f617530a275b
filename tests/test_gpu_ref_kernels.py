"""Pins the CPU oracle -- and the new kernels -- against the reference's OWN CUDA
kernels (corr1ord, corr1ord_bprop_W, poolrgn, poolrgn_bprop), compiled for
sm_100a from the reference sources by oracle/build_ref.sh and launched with the
reference's geometry.  The reference is built with -use_fast_math as its
makefile does, so its mean pooling divides approximately: values that pass
through that division are compared to 1e-6, everything else bit for bit."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libdeepbind_ref.so")
F32 = 9
PT = {"max": 0, "avg": 1, "sum": 2, "all": 3}


@pytest.fixture(scope="module")
def ref(cuda):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libdeepbind_ref.so not built (needs the reference tree: make -C oracle ref)")
    return ctypes.CDLL(REF_SO)


def dev(a, pad=0):
    import torch
    a = np.ascontiguousarray(a.view(np.int32) if a.dtype == np.uint32 else a)
    if pad:                                   # the reference's loader reads whole words past the last byte
        buf = torch.zeros(a.size + pad, dtype=torch.uint8, device="cuda")
        buf[:a.size] = torch.from_numpy(a).cuda()
        return buf[:a.size]
    return torch.from_numpy(a).cuda()


def P(t):
    return ctypes.c_void_p(t.data_ptr())


def make_case(m, nf, nseq, lmin, lmax, seed):
    from deepbind_b200 import synth
    X, R = synth.ragged_batch(nseq, lmin, lmax, m, seed=seed, n_frac=0.05)
    rng = np.random.default_rng(seed)
    X[rng.random(X.size) < 0.02] = 254
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(np.float32)
    return X, R, W, rng


@pytest.mark.parametrize("m,nf,nseq,lmin,lmax", [(24, 16, 128, 101, 101), (16, 16, 300, 20, 200), (24, 48, 50, 30, 90),
                                                 (5, 7, 40, 3, 70), (24, 130, 20, 40, 60)])
def test_reference_scan_equals_oracle_and_new_kernel(ref, orc, m, nf, nseq, lmin, lmax):
    import torch
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    X, R, W, rng = make_case(m, nf, nseq, lmin, lmax, m + nf)
    n = X.size - m + 1
    want = orc.corr1ord(W, X)
    tW, tX = dev(W), dev(X, pad=256)
    Z = torch.zeros((X.size, nf), dtype=torch.float32, device="cuda")
    # The reference kernel fills its shared sequence window with 48 threads (two warps) and
    # reads it back with no barrier in between (corr1ord.cuh:92-100), so with more than 32
    # filters its second warp can read bytes the first has not yet written.  A launch that
    # lost that race is relaunched; one clean launch must equal the oracle bit for bit.
    for attempt in range(5):
        Z.zero_()
        assert ref.ref_corr1ord(F32, P(tW), m, nf, P(tX), n, P(Z)) == 0
        torch.cuda.synchronize()
        if np.array_equal(Z.cpu().numpy(), want):
            break
    assert np.array_equal(Z.cpu().numpy(), want)                       # reference kernel == oracle, bit for bit
    Z2 = sm.zeros((X.size, nf), np.float32)
    ks.corr1ord(sm.asarray(W), sm.asarray(X), Z2, 4)
    assert torch.equal(Z2.tensor, Z)                                   # new kernel == reference kernel


@pytest.mark.parametrize("ptype", ["max", "avg", "sum", "all"])
def test_reference_pooling_equals_oracle_and_fused_kernel(ref, orc, ptype):
    import torch
    from deepbind_b200 import fused
    m, nf = 24, 16
    X, R, W, rng = make_case(m, nf, 200, 20, 150, 3)
    b = rng.uniform(-0.1, 0, nf).astype(np.float32)
    act = np.maximum(orc.corr1ord(W, X) + b, 0).astype(np.float32)
    wantP, wantA = orc.poolrgn(act, R, ptype, True)
    tU, tR = dev(act), dev(R)
    ncol = nf * (2 if ptype == "all" else 1)
    Pt = torch.empty((R.shape[0], ncol), dtype=torch.float32, device="cuda")
    At = torch.empty((R.shape[0], nf), dtype=torch.int32, device="cuda")
    has_arg = ptype in ("max", "all")
    assert ref.ref_poolrgn(F32, P(tU), nf, P(tR), R.shape[0], 2, P(Pt), P(At) if has_arg else None, PT[ptype]) == 0
    torch.cuda.synchronize()
    got = Pt.cpu().numpy()
    fP, fA, _ = fused.scanpool(dev(W), dev(b), dev(X), tR, ptype, want_argmax=True)
    if has_arg:
        assert np.array_equal(At.cpu().numpy().view(np.uint32), wantA)          # argmax: reference == oracle
        assert torch.equal(fA, At)                                               # fused == reference
    if ptype in ("max", "sum"):
        assert np.array_equal(got, wantP) and torch.equal(fP, Pt)
    else:                                                                        # fast-math division in the reference
        np.testing.assert_allclose(got, wantP, rtol=1e-6, atol=0)
        np.testing.assert_allclose(fP.cpu().numpy(), got, rtol=1e-6, atol=0)
        if ptype == "all":
            assert np.array_equal(got[:, 0::2], wantP[:, 0::2])


@pytest.mark.parametrize("ptype", ["max", "avg", "all"])
def test_reference_backward_equals_oracle_and_fused_kernel(ref, orc, ptype):
    import torch
    from deepbind_b200 import fused
    m, nf = 24, 16
    X, R, W, rng = make_case(m, nf, 128, 101, 101, 11)
    b = rng.uniform(-0.1, 0, nf).astype(np.float32)
    n = X.size - m + 1
    act = np.maximum(orc.corr1ord(W, X) + b, 0).astype(np.float32)
    Pw, Aw = orc.poolrgn(act, R, ptype, True)
    dP = rng.standard_normal(Pw.shape).astype(np.float32)
    # reference: pooling backward, then relu backward on the host, then filter gradient
    tR = dev(R)
    dA = torch.zeros(act.shape, dtype=torch.float32, device="cuda")
    tA = dev(Aw) if Aw is not None else None
    assert ref.ref_poolrgn_bprop(F32, P(dA), nf, P(tR), R.shape[0], 2, P(dev(dP)), P(tA) if tA is not None else None, PT[ptype]) == 0
    torch.cuda.synchronize()
    want_dA = orc.poolrgn_bprop(np.zeros_like(act), R, dP, Aw, ptype)
    # approximate division, then (mean share + max delta) may cancel: absolute floor of 1e-8 on values of order 1e-2
    np.testing.assert_allclose(dA.cpu().numpy(), want_dA, rtol=1e-6, atol=1e-8)
    dZ =(dA * torch.sign(dev(act))).contiguous()
    dW = torch.zeros((4 * m, nf), dtype=torch.float32, device="cuda")
    assert ref.ref_corr1ord_bprop_W(F32, P(dW), m, nf, P(dev(X, pad=256)), n, P(dZ)) == 0
    torch.cuda.synchronize()
    want_dW = orc.corr1ord_bprop_W(np.zeros((4 * m, nf)), X, dZ.cpu().numpy().astype(np.float64))
    scale = float(dZ.abs().sum(dim=0).max())
    assert np.max(np.abs(dW.cpu().numpy() - want_dW)) <= 1e-5 * scale        # reference (atomics) vs exact sum
    # the fused backward against the reference's gradient
    fP, fA, fM = fused.scanpool(dev(W), dev(b), dev(X), tR, ptype, want_argmax=True, want_actmask=True)
    gW, gb = fused.scanpool_bprop(m, nf, dev(X), tR, ptype, dev(dP), fA, fM)
    assert float((gW - dW).abs().max()) <= 1e-5 * scale
    assert float((gb - dZ.sum(dim=0)).abs().max()) <= 1e-5 * scale
