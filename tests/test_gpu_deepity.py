"""Parity of the deepity_smat entry points and the layer arithmetic with the CPU
oracle.  The update kernels may contract a multiply-add (the reference's build
does too), hence a few-ulp tolerance there; dense products are compared with
1e-5 relative to the magnitude of the summed terms."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_gradstep_family(cuda, orc, dtype):
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(0)
    n = 5003
    P, dP, mP = (rng.standard_normal(n).astype(dtype) for _ in range(3))
    dr = rng.uniform(1e-4, 1e-1, n).astype(dtype); mr = rng.uniform(0.5, 0.99, n).astype(dtype)
    rtol = 1e-6 if dtype == np.float32 else 1e-14
    for nesterov in (False, True):
        p, m_ = P.copy(), mP.copy()
        if nesterov:
            orc.gradstep_nesterov1(p, m_, mr); orc.gradstep_nesterov2(p, dP, dr, m_, mr)
        else:
            orc.gradstep(p, dP, dr, m_, mr)
        gP, gm = sm.asarray(P), sm.asarray(mP)
        calls = []
        ds.gradstep(gP, sm.asarray(dP), sm.asarray(dr), gm, sm.asarray(mr), grad=lambda: calls.append(1), nesterov=nesterov)
        assert calls == [1]
        np.testing.assert_allclose(gP.asnumpy().ravel(), p, rtol=rtol, atol=rtol)
        np.testing.assert_allclose(gm.asnumpy().ravel(), m_, rtol=rtol, atol=rtol)


def test_madd_bcast_maskout_zmask(cuda, orc):
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(1)
    A = rng.standard_normal((30, 12)).astype(f32); b = rng.standard_normal(3).astype(f32)
    dst0 = rng.standard_normal((30, 12)).astype(f32)
    want = dst0.copy(); orc.madd_bcast(A, b, 4, want)
    dst = sm.asarray(dst0); ds.madd_bcast(sm.asarray(A), b, 4, dst)
    np.testing.assert_allclose(dst.asnumpy(), want, rtol=1e-6, atol=1e-7)
    M = rng.random((30, 12)) > 0.5
    Aw = A.copy(); Aw[3, 3] = np.nan; M[3, 3] = False
    want = Aw.copy(); orc.maskout(M, want)
    gA = sm.asarray(Aw); ds.maskout(sm.asarray(M), gA)
    assert np.array_equal(gA.asnumpy(), want) and not np.isnan(gA.asnumpy()).any()
    Z = rng.integers(0, 3, size=(40, 5)).astype(f32)          # many ties
    Mw = np.zeros((40, 5), np.uint8); orc.calc_zmask(Z, Mw)
    gM = sm.zeros((40, 5), np.bool_); ds.calc_Zmask(sm.asarray(Z), gM)
    assert np.array_equal(gM.asnumpy(), Mw.astype(bool))


def test_feature_dropout(cuda, orc):
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(2)
    I, k, n = 3, 8, 64
    X = rng.standard_normal((n, I * k)).astype(f32)
    rate = np.array([0.0, 0.25, 0.5], f32)
    U = rng.random(n * I * k).astype(f32)
    for match in (False, True):
        Zw, Mw = orc.dropout_fp_tr(X, rate, U, matchrows=match)
        Z, M = ds.dropout_fp_train(sm.asarray(X), sm.asarray(rate), match, U=sm.asarray(U))
        assert np.array_equal(Z.asnumpy(), Zw) and np.array_equal(M.asnumpy(), Mw)
        dZ = rng.standard_normal(X.shape).astype(f32)
        assert np.array_equal(ds.dropout_bp_tr(sm.asarray(dZ), M).asnumpy(), orc.dropout_bp_tr(dZ, Mw))
    np.testing.assert_allclose(ds.dropout_fp_test(sm.asarray(X), sm.asarray(rate)).asnumpy(), orc.dropout_fp_te(X, rate), rtol=1e-7)
    np.testing.assert_allclose(ds.dropout_bp_te(sm.asarray(X), sm.asarray(rate)).asnumpy(), orc.dropout_bp_te(X, rate), rtol=1e-7)
    # library-drawn masks: per-model keep rates, row pairs share a mask
    big = np.ones((4000, I * k), f32)
    Z, M = ds.dropout_fp_train(sm.asarray(big), sm.asarray(rate), True)
    mk = M.asnumpy()
    assert np.array_equal(mk[0::2], mk[1::2]) and np.array_equal(Z.asnumpy(), mk.astype(f32))
    keep = mk.reshape(4000, I, k).mean(axis=(0, 2))
    assert np.all(np.abs(keep - (1 - rate)) < 0.02)
    Z2, M2 = ds.dropout_fp_train(sm.asarray(big), sm.asarray(rate), True)
    assert not np.array_equal(M2.asnumpy(), mk)            # the call counter advances the stream


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("I,n,k,m", [(1, 128, 32, 32), (3, 64, 16, 1), (15, 128, 48, 32), (90, 37, 16, 1)])
def test_blockwise_dots(cuda, orc, dtype, I, n, k, m):
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(I + n)
    X = rng.standard_normal((n, k * I)).astype(dtype); W = rng.standard_normal((k * I, m)).astype(dtype)
    dZ = rng.standard_normal((n, m * I)).astype(dtype)
    tol = 1e-5 if dtype == np.float32 else 1e-12

    def close(a, b, terms):
        assert np.max(np.abs(a - b)) <= tol * terms

    close(ds.blockwise_dot(sm.asarray(X), sm.asarray(W), I).asnumpy(), orc.blockwise_dot(X, W, I), k * 4)
    close(ds.blockwise_dot_nt(sm.asarray(dZ), sm.asarray(W), I).asnumpy(), orc.blockwise_dot_nt(dZ, W, I), m * 4)
    close(ds.blockwise_dot_tn(sm.asarray(X), sm.asarray(dZ), I, sm.asarray(W)).asnumpy(), orc.blockwise_dot_tn(X, dZ, I, W), n * 4)
    if I > 1:
        Xs = rng.standard_normal((n, k)).astype(dtype)
        close(ds.blockwise_dot(sm.asarray(Xs), sm.asarray(W), I).asnumpy(), orc.blockwise_dot(Xs, W, I), k * 4)


def test_blockwise_combined(cuda, orc):
    from deepbind_b200 import smat as sm, deepity_smat as ds
    rng = np.random.default_rng(4)
    I, n, m = 4, 50, 8
    X0 = rng.standard_normal((n, 32 * I)).astype(f32); X1 = rng.standard_normal((n, 16)).astype(f32)   # X1 shared
    W = rng.standard_normal((48 * I, m)).astype(f32); dZ = rng.standard_normal((n, m * I)).astype(f32)
    bc = [False, True]
    Z = ds.blockwise_dot_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(W), I, bc).asnumpy()
    assert np.max(np.abs(Z - orc.blockwise_dot_combined([X0, X1], W, I, bc))) < 1e-4
    dX = ds.blockwise_dot_nt_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(dZ), sm.asarray(W), I, bc)
    wX = orc.blockwise_dot_nt_combined([X0, X1], dZ, W, I, bc)
    assert dX[1] is None and wX[1] is None
    assert np.max(np.abs(dX[0].asnumpy() - wX[0])) < 1e-4
    dW = ds.blockwise_dot_tn_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(dZ), sm.asarray(W), I, bc).asnumpy()
    assert np.max(np.abs(dW - orc.blockwise_dot_tn_combined([X0, X1], dZ, W, I, bc))) < 1e-3
    dWm = ds.blockwise_dot_tn_combined([sm.asarray(X0), sm.asarray(X1)], sm.asarray(dZ), sm.asarray(W), I, bc, dWmask=[True, False]).asnumpy()
    assert np.max(np.abs(dWm - orc.blockwise_dot_tn_combined([X0, X1], dZ, W, I, bc, [True, False]))) < 1e-3
    assert np.all(dWm.reshape(I, 48, m)[:, 32:] == 0)


def test_layer_arithmetic(cuda, orc):
    import torch
    from deepbind_b200 import _lib, smat as sm
    dll = _lib.load(); sm.bind_stream()
    rng = np.random.default_rng(5)
    n, c = 3001, 48
    X = rng.standard_normal((n, c)).astype(f32); b = rng.standard_normal(c).astype(f32)
    tX, tb = torch.from_numpy(X).cuda(), torch.from_numpy(b).cuda()
    Z = torch.empty_like(tX)
    dll.db_bias_add(Z.data_ptr(), tX.data_ptr(), tb.data_ptr(), n, c)
    assert np.array_equal(Z.cpu().numpy(), X + b)
    A = torch.empty_like(tX); dll.db_relu(A.data_ptr(), Z.data_ptr(), Z.numel())
    assert np.array_equal(A.cpu().numpy(), np.maximum(X + b, 0))
    dZ = torch.from_numpy(rng.standard_normal((n, c)).astype(f32)).cuda()
    dX = torch.empty_like(dZ); dll.db_relu_bprop(dX.data_ptr(), dZ.data_ptr(), A.data_ptr(), A.numel())
    assert np.array_equal(dX.cpu().numpy(), dZ.cpu().numpy() * np.sign(np.maximum(X + b, 0)))
    s = torch.empty(c, dtype=torch.float32, device="cuda"); dll.db_colsum(s.data_ptr(), dX.data_ptr(), n, c)
    want = dX.cpu().numpy().astype(np.float64).sum(axis=0)
    assert np.max(np.abs(s.cpu().numpy() - want)) < 1e-5 * np.abs(dX.cpu().numpy()).sum(axis=0).max()
    L = torch.empty_like(tX); dll.db_logistic(L.data_ptr(), tX.data_ptr(), tX.numel())
    np.testing.assert_allclose(L.cpu().numpy(), orc.logistic(X.astype(np.float64)), rtol=2e-6)
    # losses
    Zp = torch.from_numpy(rng.uniform(0.01, 0.99, (n, 6)).astype(f32)).cuda()
    Y = torch.from_numpy(rng.integers(0, 2, (n, 6)).astype(f32)).cuda()
    Ym = torch.from_numpy(rng.random((n, 6)) > 0.2).cuda()
    for kind in (0, 1):
        lo = torch.empty(6, dtype=torch.float32, device="cuda"); dz = torch.empty_like(Zp)
        dll.db_loss(kind, Zp.data_ptr(), Y.data_ptr(), Ym.data_ptr(), None, n, 6, lo.data_ptr(), dz.data_ptr())
        z, y, mk = Zp.cpu().numpy().astype(np.float64), Y.cpu().numpy().astype(np.float64), Ym.cpu().numpy()
        l = (z - y) ** 2 if kind == 0 else np.log(np.maximum(1e-15, z)) * y + np.log(np.maximum(1e-15, 1 - z)) * (1 - y)
        want = (0.5 if kind == 0 else -1.0) * np.where(mk, l, 0).mean(axis=0)
        np.testing.assert_allclose(lo.cpu().numpy(), want, rtol=1e-5)
        np.testing.assert_allclose(dz.cpu().numpy(), np.where(mk, z - y, 0) / n, rtol=1e-6, atol=1e-9)
