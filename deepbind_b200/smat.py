"""Minimal device-array type for the DeepBind hot path.

``sarray`` plays the role of the reference's ``smat.sarray``
(code/libs/smat/py/smat/smat.py): a 2-D, row-major device array identified to
the native library by an opaque handle (``_ptr``).  Only what the kangaroo /
deepity extension wrappers need is here -- creation, host transfer, shape and
dtype -- not smat's numpy-like operator surface.  Device memory is owned by a
PyTorch tensor (so it can be handed to ``torch.distributed``); the native
library borrows it through ``api_wrap`` and launches on PyTorch's current
stream.
"""
import numpy as np
import torch

from . import _lib

# dtype codes of the C ABI (smat/dtypes.h:67-80)
_CODE = {np.dtype(np.bool_): 0, np.dtype(np.int8): 1, np.dtype(np.uint8): 2, np.dtype(np.int16): 3,
         np.dtype(np.uint16): 4, np.dtype(np.int32): 5, np.dtype(np.uint32): 6, np.dtype(np.int64): 7,
         np.dtype(np.uint64): 8, np.dtype(np.float32): 9, np.dtype(np.float64): 10}
# storage dtype of the backing tensor (same width; PyTorch has few unsigned kernels)
_STORE = {np.dtype(np.bool_): torch.bool, np.dtype(np.int8): torch.int8, np.dtype(np.uint8): torch.uint8,
          np.dtype(np.int16): torch.int16, np.dtype(np.uint16): torch.int16, np.dtype(np.int32): torch.int32,
          np.dtype(np.uint32): torch.int32, np.dtype(np.int64): torch.int64, np.dtype(np.uint64): torch.int64,
          np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64}
_VIEW = {np.dtype(np.uint16): np.int16, np.dtype(np.uint32): np.int32, np.dtype(np.uint64): np.int64}

uindex = np.uint32
float32 = np.float32
float64 = np.float64
uint8 = np.uint8
_default_dtype = np.dtype(np.float32)


def set_default_dtype(dt):
    global _default_dtype
    _default_dtype = np.dtype(dt)


def get_default_dtype():
    return _default_dtype


def device():
    if not torch.cuda.is_available():
        raise _lib.SmatException("deepbind_b200 needs a CUDA device; there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def bind_stream():
    """Points the native library at PyTorch's current stream."""
    _lib.load().api_set_stream(torch.cuda.current_stream().cuda_stream)


def sync():
    _lib.load().api_sync()


class sarray(object):
    """2-D row-major device array: ``shape`` (rows, cols), numpy ``dtype``."""

    def __init__(self, tensor, dtype):
        assert tensor.is_cuda and tensor.is_contiguous()
        if tensor.dim() == 1:
            tensor = tensor.reshape(-1, 1)
        assert tensor.dim() == 2
        self._t = tensor
        self.dtype = np.dtype(dtype)
        self._ptr = _lib.load().api_wrap(tensor.data_ptr(), tensor.shape[0], tensor.shape[1], _CODE[self.dtype])

    def __del__(self):
        try:
            if getattr(self, "_ptr", None):
                _lib.load().api_delete(self._ptr)
        except Exception:
            pass

    shape = property(lambda self: tuple(self._t.shape))
    size = property(lambda self: self._t.numel())
    nrow = property(lambda self: self._t.shape[0])
    ncol = property(lambda self: self._t.shape[1])
    tensor = property(lambda self: self._t)

    def data_ptr(self):
        return self._t.data_ptr()

    def asnumpy(self):
        a = self._t.cpu().numpy()
        return a.view(self.dtype) if self.dtype in _VIEW else a

    def reshape(self, shape):
        return sarray(self._t.reshape(shape), self.dtype)

    def copy(self):
        return sarray(self._t.clone(), self.dtype)

    def fill_zero(self):
        self._t.zero_()
        return self

    def __repr__(self):
        return "sarray(shape=%s, dtype=%s)" % (self.shape, self.dtype)


def asarray(a, dtype=None):
    if isinstance(a, sarray):
        return a if dtype is None or np.dtype(dtype) == a.dtype else asarray(a.asnumpy(), dtype)
    from_numpy = isinstance(a, np.ndarray)
    a = np.asarray(a, dtype=dtype)
    if a.dtype == np.float64 and dtype is None and not from_numpy:
        a = a.astype(_default_dtype)      # Python lists and scalars take the default dtype
    dt = a.dtype
    if a.ndim == 1:
        a = a.reshape(-1, 1)
    a = np.ascontiguousarray(a)
    host = a.view(_VIEW[dt]) if dt in _VIEW else a
    return sarray(torch.from_numpy(host).to(device()), dt)


def empty(shape, dtype=None):
    dt = np.dtype(dtype) if dtype is not None else _default_dtype
    if np.isscalar(shape):
        shape = (shape, 1)
    return sarray(torch.empty(tuple(shape), dtype=_STORE[dt], device=device()), dt)


def zeros(shape, dtype=None):
    dt = np.dtype(dtype) if dtype is not None else _default_dtype
    if np.isscalar(shape):
        shape = (shape, 1)
    return sarray(torch.zeros(tuple(shape), dtype=_STORE[dt], device=device()), dt)


def empty_like(A, dtype=None):
    return empty(A.shape, dtype or A.dtype)


def zeros_like(A, dtype=None):
    return zeros(A.shape, dtype or A.dtype)
