"""Pins the CPU oracle -- and the new kernels -- against the reference's OWN code for
the rows beyond the scan and pooling kernels: the host loop of corr1ord_bprop_X, the
update kernels (gradstep*), madd_bcast, maskout / calc_zmask, feature and input
dropout, and the block-diagonal products (cuBLAS batched GEMM inside the reference's
launchers).  All of it is compiled for sm_100a from the reference sources by
oracle/build_ref.sh and run here with the reference's own launch rule.

Bars.  Integer / mask / copy work and the host loop: bit for bit.  The update kernels
are nvcc-compiled from the same expressions in the reference and in the new library,
so those two agree bit for bit; the gcc oracle rounds every product separately
(-ffp-contract=off) where nvcc fuses a multiply-add, hence 2 ulp of the largest term
there.  Dropout: the reference draws from cuRAND states; the test peeks the numbers
the next launch will draw and hands them to the kernels under test, after which
masks and outputs agree bit for bit.  Dense products: 1e-5 of the summed magnitudes
(cuBLAS fixes no summation order)."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libdeepbind_ref.so")
DT = {np.float32: 9, np.float64: 10}
f32 = np.float32


@pytest.fixture(scope="module")
def ref(cuda):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libdeepbind_ref.so not built (needs the reference tree: make -C oracle ref REF=...)")
    dll = ctypes.CDLL(REF_SO)
    if not hasattr(dll, "ref_gradstep"):
        pytest.skip("oracle/_ref/libdeepbind_ref.so predates the deepity_smat entries: rebuild it")
    return dll


def dev(a):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    if a.dtype == np.bool_:
        return torch.from_numpy(a.view(np.uint8)).cuda()
    return torch.from_numpy(a).cuda()


def P(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def host(t, dtype=None):
    a = t.cpu().numpy()
    return a.view(dtype) if dtype is not None else a


def sync():
    import torch
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("m,nf,npos", [(24, 16, 700), (16, 48, 333), (5, 7, 64), (24, 130, 150)])
def test_input_gradient_host_loop(ref, orc, dtype, m, nf, npos):
    """api_corr1ord_bprop_X == the reference's host loop (corr1ord_bprop.cu:191-201) == oracle."""
    from deepbind_b200 import smat as sm, kangaroo_smat as ks
    rng = np.random.default_rng(m * nf)
    W = (rng.standard_normal((4 * m, nf)) * 0.05).astype(dtype)
    dZ = rng.standard_normal((npos, nf)).astype(dtype)
    dZ[rng.random(dZ.shape) < 0.3] = 0
    dX0 = rng.standard_normal((npos, 4)).astype(dtype)          # the operator accumulates
    want = orc.corr1ord_bprop_X(dX0.copy(), W, dZ)
    tdX = dev(dX0)
    assert ref.ref_corr1ord_bprop_X(DT[dtype], P(tdX), npos, P(dev(W)), m, nf, P(dev(dZ))) == 0
    sync()
    assert np.array_equal(host(tdX), want)                      # reference == oracle
    gdX = sm.asarray(dX0)
    ks.corr1ord_bprop_X(gdX, sm.asarray(W), sm.asarray(dZ), 4)
    assert np.array_equal(gdX.asnumpy(), host(tdX))             # new kernel == reference


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n", [1, 31, 5003, 300000, 1300000])
def test_update_kernels(ref, orc, dtype, n):
    """gradstep, gradstep_nesterov1/2 (gradstep.cu:41-72): new == reference bit for bit;
    oracle within 2 ulp of the largest term (nvcc fuses a*b - c*d, gcc does not here)."""
    from deepbind_b200 import smat as sm
    from deepbind_b200.deepity_smat import ext_dll
    rng = np.random.default_rng(n)
    P0, dP, mP0 = (rng.standard_normal(n).astype(dtype) for _ in range(3))
    dr = rng.uniform(1e-4, 1e-1, n).astype(dtype); mr = rng.uniform(0.5, 0.99, n).astype(dtype)
    ulp = np.finfo(dtype).eps
    dll = ext_dll()

    def col(a):
        return sm.asarray(a.reshape(-1, 1))

    for kind in ("plain", "nesterov1", "nesterov2"):
        rP, rm = dev(P0), dev(mP0)
        gP, gm = col(P0), col(mP0)
        gdP, gdr, gmr = col(dP), col(dr), col(mr)           # named: a handle lives as long as its sarray
        oP, om = P0.copy(), mP0.copy()
        if kind == "plain":
            assert ref.ref_gradstep(DT[dtype], n, P(rP), P(dev(dP)), P(dev(dr)), P(rm), P(dev(mr))) == 0
            dll.api_gradstep(gP._ptr, gdP._ptr, gdr._ptr, gm._ptr, gmr._ptr)
            orc.gradstep(oP, dP, dr, om, mr)
        elif kind == "nesterov1":
            assert ref.ref_gradstep_nesterov1(DT[dtype], n, P(rP), P(rm), P(dev(mr))) == 0
            dll.api_gradstep_nesterov1(gP._ptr, gm._ptr, gmr._ptr)
            orc.gradstep_nesterov1(oP, om, mr)
        else:
            assert ref.ref_gradstep_nesterov2(DT[dtype], n, P(rP), P(dev(dP)), P(dev(dr)), P(rm), P(dev(mr))) == 0
            dll.api_gradstep_nesterov2(gP._ptr, gdP._ptr, gdr._ptr, gm._ptr, gmr._ptr)
            orc.gradstep_nesterov2(oP, dP, dr, om, mr)
        sync()
        assert np.array_equal(gP.asnumpy().ravel(), host(rP)), kind          # new == reference
        assert np.array_equal(gm.asnumpy().ravel(), host(rm)), kind
        bound = 2 * ulp * (np.abs(P0) + np.abs(mP0) + np.abs(dP)).max()
        assert np.max(np.abs(host(rP) - oP)) <= bound, kind                  # reference vs oracle
        assert np.max(np.abs(host(rm) - om)) <= bound, kind


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_madd_bcast_and_masks(ref, orc, dtype):
    """madd_bcast.cu:41-47, maskout.cu:41-67."""
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(7)
    for rows, cols, nb, k in [(30, 12, 3, 4), (257, 96, 6, 16), (1000, 90, 90, 1), (5, 8, 1, 40)]:
        A = rng.standard_normal((rows, cols)).astype(dtype); b = rng.standard_normal(nb).astype(dtype)
        d0 = rng.standard_normal((rows, cols)).astype(dtype)
        want = d0.copy(); orc.madd_bcast(A, b, k, want)
        rd = dev(d0)
        assert ref.ref_madd_bcast(DT[dtype], P(dev(A)), P(dev(b)), P(rd), A.size, nb, k) == 0
        gd = sm.asarray(d0); ds.madd_bcast(sm.asarray(A), b, k, gd)
        sync()
        assert np.array_equal(gd.asnumpy(), host(rd))                        # new == reference
        assert np.max(np.abs(host(rd) - want)) <= 2 * np.finfo(dtype).eps * (np.abs(d0).max() + np.abs(A).max() * np.abs(b).max())
        # maskout: clears where the mask is false, NaN included
        M = rng.random((rows, cols)) > 0.5
        Aw = A.copy(); Aw[0, 0] = np.nan; M[0, 0] = False; Aw[rows - 1, cols - 1] = np.nan; M[rows - 1, cols - 1] = True
        want = Aw.copy(); orc.maskout(M, want)
        rA = dev(Aw)
        assert ref.ref_maskout(DT[dtype], P(dev(M)), P(rA), Aw.size) == 0
        gA = sm.asarray(Aw); ds.maskout(sm.asarray(M), gA)
        sync()
        assert np.array_equal(host(rA), want, equal_nan=True) and np.array_equal(gA.asnumpy(), want, equal_nan=True)
    # calc_zmask: the stronger row of every pair, the first on ties
    for rows, cols in [(40, 5), (2, 1), (600, 90)]:
        Z = rng.integers(0, 3, size=(rows, cols)).astype(dtype)
        Mw = np.zeros((rows, cols), np.uint8); orc.calc_zmask(Z, Mw)
        import torch
        rM = torch.zeros((rows, cols), dtype=torch.uint8, device="cuda")
        assert ref.ref_calc_zmask(DT[dtype], P(dev(Z)), P(rM), rows, cols) == 0
        gM = sm.zeros((rows, cols), np.bool_); ds.calc_Zmask(sm.asarray(Z), gM)
        sync()
        assert np.array_equal(host(rM), Mw) and np.array_equal(gM.asnumpy(), Mw.astype(bool))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("match", [False, True])
def test_feature_dropout_with_the_reference_draws(ref, orc, dtype, match):
    """dropout.cu:41-162.  The uniforms the reference launch is about to draw are read
    first and given to the oracle and to api_dropout_fp_tr_u."""
    import torch
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(11)
    I, k, n = 3, 8, 640
    X = rng.standard_normal((n, I * k)).astype(dtype)
    rate = np.array([0.0, 0.25, 0.5], dtype)
    count = X.size // 2 if match else X.size
    assert ref.ref_seed(1234) == 0
    U = torch.empty(count, dtype=torch.float32, device="cuda")
    assert ref.ref_peek_uniforms(P(U), count) == 0
    rZ = torch.empty(X.shape, dtype=torch.float32 if dtype == f32 else torch.float64, device="cuda")
    rM = torch.zeros(X.shape, dtype=torch.uint8, device="cuda")
    assert ref.ref_dropout_fp_tr(DT[dtype], P(dev(X)), P(dev(rate)), P(rZ), P(rM), X.size, I, k, int(match)) == 0
    sync()
    Un = host(U)
    assert 0.0 < Un.min() and Un.max() <= 1.0 and abs(Un.mean() - 0.5) < 0.02
    Zw, Mw = orc.dropout_fp_tr(X, rate, Un, matchrows=match)
    assert np.array_equal(host(rM).astype(bool), Mw) and np.array_equal(host(rZ), Zw)       # reference == oracle
    Z, M = ds.dropout_fp_train(sm.asarray(X), sm.asarray(rate), match, U=sm.asarray(Un))
    assert np.array_equal(M.asnumpy(), Mw) and np.array_equal(Z.asnumpy(), host(rZ))         # new == reference
    keep = Mw.reshape(n, I, k).mean(axis=(0, 2))
    assert np.all(np.abs(keep - (1 - rate.astype(np.float64))) < 0.03)
    # a second launch draws fresh numbers (the states advance)
    rM2 = torch.zeros_like(rM)
    assert ref.ref_dropout_fp_tr(DT[dtype], P(dev(X)), P(dev(rate)), P(rZ), P(rM2), X.size, I, k, int(match)) == 0
    sync()
    assert not np.array_equal(host(rM2), host(rM))
    # backward and test-mode passes
    dZ = rng.standard_normal(X.shape).astype(dtype)
    rdX = torch.empty_like(rZ)
    assert ref.ref_dropout_bp_tr(DT[dtype], P(dev(dZ)), P(rM), P(rdX), X.size) == 0
    sync()
    assert np.array_equal(host(rdX), orc.dropout_bp_tr(dZ, Mw))
    assert np.array_equal(ds.dropout_bp_tr(sm.asarray(dZ), M).asnumpy(), host(rdX))
    assert ref.ref_dropout_fp_te(DT[dtype], P(dev(X)), P(dev(rate)), P(rZ), X.size, I, k) == 0
    sync()
    assert np.array_equal(host(rZ), orc.dropout_fp_te(X, rate))
    assert np.array_equal(ds.dropout_fp_test(sm.asarray(X), sm.asarray(rate)).asnumpy(), host(rZ))
    assert ref.ref_dropout_bp_te(DT[dtype], P(dev(dZ)), P(dev(rate)), P(rdX), X.size, I, k) == 0
    sync()
    assert np.array_equal(host(rdX), orc.dropout_bp_te(dZ, rate))
    assert np.array_equal(ds.dropout_bp_te(sm.asarray(dZ), sm.asarray(rate)).asnumpy(), host(rdX))


def test_input_dropout_with_the_reference_draws(ref, orc):
    """dropoutord.cu:41-60: padding (255) is never dropped, dropped bases become 254."""
    import torch
    from deepbind_b200 import smat as sm, kangaroo_smat as ks, synth
    X, R = synth.ragged_batch(200, 20, 120, 24, seed=3, n_frac=0.05)
    X = X.reshape(-1, 1)
    rate = 0.3
    assert ref.ref_seed(99) == 0
    U = torch.empty(X.size, dtype=torch.float32, device="cuda")
    assert ref.ref_peek_uniforms(P(U), X.size) == 0
    rZ = torch.empty(X.shape, dtype=torch.uint8, device="cuda"); rM = torch.zeros(X.shape, dtype=torch.uint8, device="cuda")
    assert ref.ref_dropoutord_fp_tr(P(dev(X)), P(rZ), P(rM), X.size, ctypes.c_float(rate)) == 0
    sync()
    Un = host(U)
    Zw, Mw = orc.dropoutord_fp_tr(X, Un, rate)
    assert np.array_equal(host(rZ).ravel(), Zw) and np.array_equal(host(rM).ravel().astype(bool), Mw)
    Z, M = ks.dropoutord_fp_train(sm.asarray(X), rate, U=sm.asarray(Un.reshape(-1, 1)))
    assert np.array_equal(Z.asnumpy(), host(rZ)) and np.array_equal(M.asnumpy().astype(bool), host(rM).astype(bool))
    assert np.all(host(rZ)[X == 255] == 255) and (host(rZ) == 254).sum() > 0.2 * (X < 4).sum()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("I,n,k,m", [(1, 128, 32, 32), (3, 64, 16, 1), (15, 128, 48, 32), (90, 37, 16, 1), (5, 200, 32, 32)])
def test_blockwise_products(ref, orc, dtype, I, n, k, m):
    """blockwise_dot.cu:42-154 (cuBLAS batched GEMM in the reference)."""
    import torch
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(I * 1000 + n)
    X = rng.standard_normal((n, k * I)).astype(dtype); W = rng.standard_normal((k * I, m)).astype(dtype)
    dZ = rng.standard_normal((n, m * I)).astype(dtype)
    tdt = torch.float32 if dtype == f32 else torch.float64
    tol = 1e-5 if dtype == f32 else 1e-12

    def close(a, b, terms):
        assert np.max(np.abs(a - b)) <= tol * terms

    rZ = torch.zeros((n, m * I), dtype=tdt, device="cuda")
    assert ref.ref_blockwise_dot(DT[dtype], I, n, m, k, 0, P(dev(X)), P(dev(W)), P(rZ)) == 0
    sync()
    close(host(rZ), orc.blockwise_dot(X, W, I), k * 4)
    close(ds.blockwise_dot(sm.asarray(X), sm.asarray(W), I).asnumpy(), host(rZ), k * 4)
    rdX = torch.zeros((n, k * I), dtype=tdt, device="cuda")
    assert ref.ref_blockwise_dot_nt(DT[dtype], I, n, m, k, P(dev(dZ)), P(dev(W)), P(rdX)) == 0
    sync()
    close(host(rdX), orc.blockwise_dot_nt(dZ, W, I), m * 4)
    close(ds.blockwise_dot_nt(sm.asarray(dZ), sm.asarray(W), I).asnumpy(), host(rdX), m * 4)
    rdW = torch.zeros((k * I, m), dtype=tdt, device="cuda")
    assert ref.ref_blockwise_dot_tn(DT[dtype], I, n, m, k, 0, P(dev(X)), P(dev(dZ)), P(rdW)) == 0
    sync()
    close(host(rdW), orc.blockwise_dot_tn(X, dZ, I, W), n * 4)
    close(ds.blockwise_dot_tn(sm.asarray(X), sm.asarray(dZ), I, sm.asarray(W)).asnumpy(), host(rdW), n * 4)
    if I > 1:                                                   # one input shared by all models
        Xs = rng.standard_normal((n, k)).astype(dtype)
        assert ref.ref_blockwise_dot(DT[dtype], I, n, m, k, 1, P(dev(Xs)), P(dev(W)), P(rZ)) == 0
        sync()
        close(host(rZ), orc.blockwise_dot(Xs, W, I), k * 4)
        close(ds.blockwise_dot(sm.asarray(Xs), sm.asarray(W), I).asnumpy(), host(rZ), k * 4)


def test_blockwise_combined_products(ref, orc):
    """blockwise_dot.cu:157-260: two inputs (pooled features per model, 16 shared
    feature columns) against one stacked weight matrix of p = 48 rows per model."""
    import torch
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(4)
    I, n, m, p = 4, 50, 8, 48
    X0 = rng.standard_normal((n, 32 * I)).astype(f32); X1 = rng.standard_normal((n, 16)).astype(f32)
    W = rng.standard_normal((p * I, m)).astype(f32); dZ = rng.standard_normal((n, m * I)).astype(f32)
    bc = [False, True]
    tW, tdZ = dev(W), dev(dZ)
    rZ = torch.zeros((n, m * I), dtype=torch.float32, device="cuda")
    assert ref.ref_blockwise_dot_combined(9, I, 0, 0, n, m, 32, p, P(dev(X0)), P(tW), P(rZ)) == 0
    assert ref.ref_blockwise_dot_combined(9, I, 32, 1, n, m, 16, p, P(dev(X1)), P(tW), P(rZ)) == 0
    sync()
    want = orc.blockwise_dot_combined([X0, X1], W, I, bc)
    assert np.max(np.abs(host(rZ) - want)) < 1e-5 * 48 * 4
    got = ds.blockwise_dot_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(W), I, bc).asnumpy()
    assert np.max(np.abs(got - host(rZ))) < 1e-5 * 48 * 4
    rdX = torch.zeros((n, 32 * I), dtype=torch.float32, device="cuda")
    assert ref.ref_blockwise_dot_nt_combined(9, I, 0, n, m, 32, p, P(rdX), P(tW), P(tdZ)) == 0
    sync()
    wX = orc.blockwise_dot_nt_combined([X0, X1], dZ, W, I, bc)
    assert np.max(np.abs(host(rdX) - wX[0])) < 1e-5 * m * 4
    gX = ds.blockwise_dot_nt_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(dZ), sm.asarray(W), I, bc)
    assert np.max(np.abs(gX[0].asnumpy() - host(rdX))) < 1e-5 * m * 4
    rdW = torch.zeros((p * I, m), dtype=torch.float32, device="cuda")
    assert ref.ref_blockwise_dot_tn_combined(9, I, 0, 0, n, m, 32, p, P(dev(X0)), P(rdW), P(tdZ)) == 0
    assert ref.ref_blockwise_dot_tn_combined(9, I, 32, 1, n, m, 16, p, P(dev(X1)), P(rdW), P(tdZ)) == 0
    sync()
    wW = orc.blockwise_dot_tn_combined([X0, X1], dZ, W, I, bc)
    # with a shared input the reference's batched product leaves each model's 16 feature rows
    # holding that model's own sum, as the oracle states it
    assert np.max(np.abs(host(rdW) - wW)) < 1e-5 * n * 4
    gW = ds.blockwise_dot_tn_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(dZ), sm.asarray(W), I, bc).asnumpy()
    assert np.max(np.abs(gW - host(rdW))) < 1e-5 * n * 4
