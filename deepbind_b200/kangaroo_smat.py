"""Python side of the kangaroo_smat boundary.

Same function names, argument order and meaning as the reference's
``kangaroo/_ext/kangaroo_smat.py`` (code/libs/kangaroo/kangaroo/_ext/kangaroo_smat.py:85-150),
bound to libdeepbind_b200.so.  Arguments are :class:`deepbind_b200.smat.sarray`.
"""
from ctypes import byref

import numpy as np

from . import _lib
from .smat import empty, empty_like, bind_stream, uindex

c_pm_zero_output = 0
str2pooltype = {"max": 0, "avg": 1, "sum": 2, "all": 3}


def ext_dll():
    dll = _lib.load()
    bind_stream()
    return dll


def _corr_options(nchannel):
    options = _lib.c_corr1ord_options_t()
    options.padmode = c_pm_zero_output
    options.nchannel = nchannel
    return options


def corr1ord(W, X, Z, nchannel):
    """Cross-correlates the filters W [(M*nchannel), P] with the ordinal vector X
    (uint8; 0..nchannel-1, 254 = dropped, anything else = "all ordinals").
    Writes Z [N, P]; the final M-1 rows of Z are left as the caller set them."""
    ext_dll().api_corr1ord(W._ptr, X._ptr, Z._ptr, byref(_corr_options(nchannel)))


def corr1ord_bprop_W(dW, X, dZ, nchannel):
    """Accumulates the filter gradient of corr1ord into dW (caller zeroes dW)."""
    ext_dll().api_corr1ord_bprop_W(dW._ptr, X._ptr, dZ._ptr, byref(_corr_options(nchannel)))


def corr1ord_bprop_X(dX, W, dZ, nchannel):
    """Accumulates the input gradient of corr1ord into dX [N, nchannel]."""
    ext_dll().api_corr1ord_bprop_X(dX._ptr, W._ptr, dZ._ptr, byref(_corr_options(nchannel)))


def poolrgn(unpooledmaps, regions, ptype, want_argmax=False):
    noutputs = 2 if ptype == "all" else 1
    options = _lib.c_poolrgn_options_t()
    options.ptype = str2pooltype[ptype]
    nregion = regions.shape[0]
    nfeaturemap = unpooledmaps.shape[1]
    pooledmaps = empty((nregion, nfeaturemap * noutputs), dtype=unpooledmaps.dtype)
    pooledmaps_argmax = empty((nregion, nfeaturemap), dtype=uindex) if (ptype in ("max", "all") and want_argmax) else None
    ext_dll().api_poolrgn(unpooledmaps._ptr, regions._ptr, pooledmaps._ptr,
                          pooledmaps_argmax._ptr if pooledmaps_argmax is not None else None, byref(options))
    if want_argmax:
        return pooledmaps, pooledmaps_argmax
    return pooledmaps, None


def poolrgn_bprop(unpooledmaps, regions, pooledmaps, pooledmaps_argmax, ptype):
    options = _lib.c_poolrgn_options_t()
    options.ptype = str2pooltype[ptype]
    argmax_ptr = pooledmaps_argmax._ptr if (pooledmaps_argmax is not None) and (ptype in ("max", "all")) else None
    ext_dll().api_poolrgn_bprop(unpooledmaps._ptr, regions._ptr, pooledmaps._ptr, argmax_ptr, byref(options))


def dropoutord_fp_train(X, rate, U=None):
    """Returns (Z, M): Z = X with dropped bases set to 254, M the keep mask.
    ``U`` optionally supplies the uniform draws (float32, one per element)."""
    Z = empty_like(X)
    M = empty(X.shape, dtype=np.bool_)
    if U is None:
        ext_dll().api_dropoutord_fp_tr(X._ptr, Z._ptr, M._ptr, rate)
    else:
        ext_dll().api_dropoutord_fp_tr_u(X._ptr, U._ptr, Z._ptr, M._ptr, rate)
    return Z, M


def autotune():
    ext_dll().api_autotune()
