"""Bias, rectifier, logistic and the loss formulas against the reference's OWN element-wise
kernels.  The reference's layer nodes are Python over smat arrays
(deepity/std/elemwise.py:71-82,109-113,162-180, softmax.py:50-61, loss.py:98-155): `X + b`,
`maximum(0, X)`, `dZ * sign(Z)`, `logistic(X)`, `log(maximum(1e-15, Z)) * Y + ...`, `(Z - Y)**2`,
`Z - Y`, `dZ *= 1/nrow`.  Each of those is one launch of smat's element-wise kernels
(smat_cuda/elemwise2.cu, elemwise3.cu), which oracle/build_ref.sh compiles for sm_100a from the
reference sources with the reference's -use_fast_math.  The tests run the same chain of
launches the Python expressions would issue and compare the CPU oracle and the new kernels.

Bars.  Adds, maxima, sign products, differences and the 1/nrow scaling: bit for bit.  The
logistic: the reference evaluates 1/(1+__expf(-x)) with an approximate division, the new kernel
expf and an IEEE division: 4e-7 absolute on values in (0, 1).  The log-likelihood: __logf
against logf, 2e-6 of the largest term.  Means over the minibatch: 1e-6 relative (the
reference's reduction order is its own)."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libdeepbind_ref.so")
F32 = 9


@pytest.fixture(scope="module")
def ref(cuda):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libdeepbind_ref.so not built (needs the reference tree: make -C oracle ref REF=...)")
    dll = ctypes.CDLL(REF_SO)
    if not hasattr(dll, "ref_elemwise3"):
        pytest.skip("oracle/_ref/libdeepbind_ref.so predates the element-wise entries: rebuild it")
    dll.ref_elemwise3.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_uint, ctypes.c_uint,
                                  ctypes.c_void_p, ctypes.c_float, ctypes.c_uint, ctypes.c_uint, ctypes.c_void_p]
    dll.ref_elemwise2.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint, ctypes.c_uint]
    return dll


class Smat(object):
    """The handful of smat operations the layer nodes use, each one launch of the reference's kernels."""

    def __init__(self, dll):
        import torch
        self.dll, self.torch = dll, torch
        self.oc = {k: dll.ref_opcode(k.encode()) for k in ("add", "sub", "mul", "maxe", "log", "sigm", "sign", "sqr")}
        assert all(v >= 0 for v in self.oc.values())

    def _bin(self, op, a, b):
        torch = self.torch
        at, bt = torch.is_tensor(a), torch.is_tensor(b)
        shp = tuple(max(x, y) for x, y in zip(a.shape if at else (1, 1), b.shape if bt else (1, 1)))
        c = torch.empty(shp, dtype=torch.float32, device="cuda")
        rc = self.dll.ref_elemwise3(self.oc[op], F32, a.data_ptr() if at else None, 0.0 if at else float(a),
                                    a.shape[0] if at else 1, a.shape[1] if at else 1,
                                    b.data_ptr() if bt else None, 0.0 if bt else float(b),
                                    b.shape[0] if bt else 1, b.shape[1] if bt else 1, c.data_ptr())
        assert rc == 0
        return c

    def _un(self, op, a):
        b = self.torch.empty_like(a)
        assert self.dll.ref_elemwise2(self.oc[op], F32, a.data_ptr(), b.data_ptr(), a.shape[0], a.shape[1]) == 0
        return b

    add = lambda self, a, b: self._bin("add", a, b)
    sub = lambda self, a, b: self._bin("sub", a, b)
    mul = lambda self, a, b: self._bin("mul", a, b)
    maximum = lambda self, a, b: self._bin("maxe", a, b)
    log = lambda self, a: self._un("log", a)
    logistic = lambda self, a: self._un("sigm", a)
    sign = lambda self, a: self._un("sign", a)
    square = lambda self, a: self._un("sqr", a)


def _data(nrow, ncol, seed):
    import torch
    g = np.random.default_rng(seed)
    X = g.standard_normal((nrow, ncol)).astype(np.float32)
    X[g.random((nrow, ncol)) < 0.1] = 0.0                       # exact zeros: the rectifier's edge
    X[0, 0], X[0, 1 % ncol] = -0.0, 0.0
    return torch.from_numpy(X).cuda(), g


@pytest.mark.parametrize("nrow,ncol", [(1, 1), (37, 16), (300, 48), (2048, 33)])
def test_bias_and_rectifier_forward_and_backward(ref, orc, nrow, ncol):
    import torch
    from deepbind_b200 import _lib
    dll = _lib.load()
    sm = Smat(ref)
    X, g = _data(nrow, ncol, 3)
    b = torch.from_numpy(g.standard_normal((1, ncol)).astype(np.float32)).cuda()
    dZ = torch.from_numpy(g.standard_normal((nrow, ncol)).astype(np.float32)).cuda()
    # elemwise.py:171  Z = X + b (row vector broadcast)
    want = sm.add(X, b)
    got = torch.empty_like(X)
    dll.db_bias_add(got.data_ptr(), X.data_ptr(), b.data_ptr(), nrow, ncol)
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    np.testing.assert_array_equal(orc.bias_add(X.cpu().numpy(), b.cpu().numpy().ravel()).view(np.uint32), want.cpu().numpy().view(np.uint32))
    # elemwise.py:77  Z = maximum(0, X)
    relu_ref = sm.maximum(0.0, want)
    relu_new = torch.empty_like(X)
    dll.db_relu(relu_new.data_ptr(), want.data_ptr(), want.numel())
    assert torch.equal(relu_new, relu_ref) and bool((relu_new >= 0).all())
    np.testing.assert_array_equal(orc.relu(want.cpu().numpy()), relu_ref.cpu().numpy())
    # elemwise.py:78  dX = dZ * sign(Z), Z the rectified value
    dX_ref = sm.mul(dZ, sm.sign(relu_ref))
    dX_new = torch.empty_like(X)
    dll.db_relu_bprop(dX_new.data_ptr(), dZ.data_ptr(), relu_ref.data_ptr(), dZ.numel())
    assert torch.equal(dX_new, dX_ref)
    np.testing.assert_array_equal(orc.relu_bprop(dZ.cpu().numpy(), relu_ref.cpu().numpy()), dX_ref.cpu().numpy())


@pytest.mark.parametrize("nrow,ncol", [(64, 1), (500, 7)])
def test_logistic_and_losses(ref, orc, nrow, ncol):
    import torch
    from deepbind_b200 import _lib
    dll = _lib.load()
    sm = Smat(ref)
    X, g = _data(nrow, ncol, 5)
    X = X * 4
    X[1, 0], X[2, 0] = 40.0, -40.0                               # saturated outputs: the 1e-15 floor of the likelihood
    Y = torch.from_numpy((g.random((nrow, ncol)) < 0.5).astype(np.float32)).cuda()
    # softmax.py:50-61 with one column per model: Z = logistic(X)
    Z_ref = sm.logistic(X)
    Z_new = torch.empty_like(X)
    dll.db_logistic(Z_new.data_ptr(), X.data_ptr(), X.numel())
    assert float((Z_new - Z_ref).abs().max()) <= 4e-7
    np.testing.assert_allclose(orc.logistic(X.cpu().numpy()), Z_ref.cpu().numpy(), atol=4e-7, rtol=0)
    # loss.py:140-145  L = log(maximum(1e-15,Z))*Y + log(maximum(1e-15,1-Z))*(1-Y); mean over rows; negated
    Z = Z_new
    L_ref = sm.add(sm.mul(sm.log(sm.maximum(1e-15, Z)), Y), sm.mul(sm.log(sm.maximum(1e-15, sm.sub(1.0, Z))), sm.sub(1.0, Y)))
    nll_ref = -(L_ref.double().mean(dim=0))
    loss = torch.empty(ncol, dtype=torch.float32, device="cuda")
    dZ = torch.empty_like(Z)
    dll.db_loss(1, Z.data_ptr(), Y.data_ptr(), None, None, nrow, ncol, loss.data_ptr(), dZ.data_ptr())
    scale = float(L_ref.abs().max())
    assert float((loss.double() - nll_ref).abs().max()) <= 2e-6 * scale
    want_o = orc.loss("nll", Z.cpu().numpy(), Y.cpu().numpy())[0]
    np.testing.assert_allclose(want_o, nll_ref.cpu().numpy(), atol=2e-6 * scale, rtol=0)
    # loss.py:109-112  dZ = Z - Y, then dZ *= 1/nrow
    dZ_ref = sm.mul(sm.sub(Z, Y), float(np.float32(1.0) / np.float32(nrow)))
    assert torch.equal(dZ, dZ_ref)
    # loss.py:131-134  mse: 0.5 * mean((Z - Y)**2)
    T = torch.from_numpy(g.standard_normal((nrow, ncol)).astype(np.float32)).cuda()
    sq_ref = sm.square(sm.sub(X, T))
    mse_ref = 0.5 * sq_ref.double().mean(dim=0)
    dll.db_loss(0, X.data_ptr(), T.data_ptr(), None, None, nrow, ncol, loss.data_ptr(), dZ.data_ptr())
    assert float(((loss.double() - mse_ref).abs() / mse_ref).max()) <= 1e-6
    assert torch.equal(dZ, sm.mul(sm.sub(X, T), float(np.float32(1.0) / np.float32(nrow))))
    np.testing.assert_allclose(orc.loss("mse", X.cpu().numpy(), T.cpu().numpy())[0], mse_ref.cpu().numpy(), rtol=1e-6)
