"""ctypes binding of libdeepbind_b200.so.

Every exported function is called through :class:`_SafeFunc`, which reads the
library's error string after the call and raises :class:`SmatException`, the
way the reference's ``safe_dll_func`` does
(code/libs/smat/py/smat/smat_dll.py:160-183).  There is no fallback: if the
shared library is missing or cannot be loaded, importing the compute modules
fails with the build command to run.
"""
import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_size_t,
                    c_uint32, c_uint64, c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libdeepbind_b200.so")


class SmatException(Exception):
    pass


class c_shape_t(Structure):
    _fields_ = [("x", c_int32), ("y", c_int32), ("z", c_int32)]


class c_smat(Structure):
    # Prefix of the native handle (smat_dll.py:85-92); never allocated in Python.
    _fields_ = [("vtype", c_int), ("dtype", c_int), ("shape", c_shape_t), ("strides", c_shape_t)]


c_smat_p = POINTER(c_smat)


class c_corr1ord_options_t(Structure):
    _fields_ = [("padmode", c_int), ("nchannel", c_uint32)]


class c_ministep_args(Structure):
    """struct db_ministep_args of include/deepbind_b200.h."""
    _fields_ = [(k, ctypes.c_uint32) for k in ("nmodel", "nfilt", "m", "ptype", "hidden", "loss_kind", "strand_pairs", "B",
                                               "max_rows", "npos")] + \
               [("X", ctypes.c_void_p), ("X_stride", ctypes.c_size_t), ("R", ctypes.c_void_p), ("R_stride", ctypes.c_size_t),
                ("Y", ctypes.c_void_p), ("Y_stride", ctypes.c_size_t), ("dropmask", ctypes.c_void_p), ("mask_stride", ctypes.c_size_t),
                ("counters", ctypes.c_void_p), ("order", ctypes.c_void_p), ("nbatch", ctypes.c_uint32)] + \
               [(k, ctypes.c_void_p) for k in ("P", "PL", "mP", "dP", "drate", "mrate", "decay")] + \
               [(k, ctypes.c_uint32) for k in ("off_Wscan", "off_bscan", "off_W1", "off_b1", "off_W2", "off_b2")] + \
               [("loss", ctypes.c_void_p), ("status", ctypes.c_void_p)]


class c_poolrgn_options_t(Structure):
    _fields_ = [("ptype", c_int)]


P = c_void_p
_PROTOTYPES = {
    # name: (restype, argtypes)
    "api_get_last_error": (c_char_p, []),
    "api_clear_last_error": (None, []),
    "api_sync": (None, []),
    "api_set_stream": (None, [c_void_p]),
    "api_get_stream": (c_void_p, []),
    "api_device_count": (c_int, []),
    "api_set_device": (None, [c_int]),
    "api_empty": (c_smat_p, [POINTER(c_shape_t), c_int]),
    "api_zeros": (c_smat_p, [POINTER(c_shape_t), c_int]),
    "api_wrap": (c_smat_p, [c_void_p, c_int, c_int, c_int]),
    "api_delete": (None, [c_smat_p]),
    "api_nrow": (c_int32, [c_smat_p]),
    "api_ncol": (c_int32, [c_smat_p]),
    "api_size": (c_size_t, [c_smat_p]),
    "api_dtype": (c_int, [c_smat_p]),
    "api_data": (c_void_p, [c_smat_p]),
    "api_copy_from": (None, [c_smat_p, c_void_p, c_int32, c_int32]),
    "api_copy_to": (None, [c_smat_p, c_void_p, c_int32, c_int32]),
    "api_fill_zero": (None, [c_smat_p]),
    "api_set_seed": (None, [c_uint64]),
    "api_launch_count": (c_uint64, []),
    "db_reserve_scratch": (None, [c_size_t]),
    "db_scratch_bytes": (c_size_t, []),
    "register_ext": (None, []),
    "api_autotune": (None, []),
    "api_corr1ord": (None, [c_smat_p, c_smat_p, c_smat_p, POINTER(c_corr1ord_options_t)]),
    "api_corr1ord_bprop_W": (None, [c_smat_p, c_smat_p, c_smat_p, POINTER(c_corr1ord_options_t)]),
    "api_corr1ord_bprop_X": (None, [c_smat_p, c_smat_p, c_smat_p, POINTER(c_corr1ord_options_t)]),
    "api_poolrgn": (None, [c_smat_p, c_smat_p, c_smat_p, c_smat_p, POINTER(c_poolrgn_options_t)]),
    "api_poolrgn_bprop": (None, [c_smat_p, c_smat_p, c_smat_p, c_smat_p, POINTER(c_poolrgn_options_t)]),
    "api_dropoutord_fp_tr": (None, [c_smat_p, c_smat_p, c_smat_p, c_float]),
    "api_dropoutord_fp_tr_u": (None, [c_smat_p, c_smat_p, c_smat_p, c_smat_p, c_float]),
    "api_gradstep": (None, [c_smat_p] * 5),
    "api_gradstep_nesterov1": (None, [c_smat_p] * 3),
    "api_gradstep_nesterov2": (None, [c_smat_p] * 5),
    "api_madd_bcast": (None, [c_smat_p, c_smat_p, c_uint32, c_smat_p]),
    "api_maskout": (None, [c_smat_p, c_smat_p]),
    "api_calc_zmask": (None, [c_smat_p, c_smat_p]),
    "api_dropout_fp_tr": (None, [c_smat_p, c_smat_p, c_smat_p, c_smat_p, c_int]),
    "api_dropout_fp_tr_u": (None, [c_smat_p, c_smat_p, c_smat_p, c_smat_p, c_smat_p, c_int]),
    "api_dropout_fp_te": (None, [c_smat_p] * 3),
    "api_dropout_bp_tr": (None, [c_smat_p] * 3),
    "api_dropout_bp_te": (None, [c_smat_p] * 3),
    "api_blockwise_dot": (None, [c_int, c_smat_p, c_smat_p, c_smat_p]),
    "api_blockwise_dot_nt": (None, [c_int, c_smat_p, c_smat_p, c_smat_p]),
    "api_blockwise_dot_tn": (None, [c_int, c_smat_p, c_smat_p, c_smat_p]),
    "api_blockwise_dot_combined": (None, [c_int, c_int, c_int, c_smat_p, c_smat_p, c_smat_p]),
    "api_blockwise_dot_nt_combined": (None, [c_int, c_int, c_int, c_smat_p, c_smat_p, c_smat_p]),
    "api_blockwise_dot_tn_combined": (None, [c_int, c_int, c_int, c_smat_p, c_smat_p, c_smat_p]),
    "db_bias_add": (None, [P, P, P, c_uint32, c_uint32]),
    "db_relu": (None, [P, P, c_size_t]),
    "db_relu_bprop": (None, [P, P, P, c_size_t]),
    "db_colsum": (None, [P, P, c_uint32, c_uint32]),
    "db_colsum_static": (None, [P, P, c_uint32, c_uint32]),
    "db_logistic": (None, [P, P, c_size_t]),
    "db_strand_max": (None, [P, P, c_uint32, c_uint32]),
    "db_randn": (None, [P, c_size_t]),
    "db_loss": (None, [c_int, P, P, P, P, c_uint32, c_uint32, P, P]),
    "db_l1_decay": (None, [P, P, P, c_size_t]),
    "db_fadd_probe": (c_uint64, [P, c_uint32]),
    "db_dropout_mask": (None, [P, c_uint32, c_uint32, P, c_uint32, c_int, P]),
    "db_minibatch_fetch": (None, [P, P, c_uint32, P, P, c_size_t, P, P, c_size_t, P, P, c_size_t]),
    "db_head_max_batch": (c_uint32, [c_uint32, c_uint32]),
    "db_head_train": (None, [c_uint32, c_uint32, c_uint32, c_int, c_int, c_uint32, P, P, P, P, P, P, P, P, P, P, P, P, P]),
    "db_ministep_supported": (c_int, [POINTER(c_ministep_args)]),
    "db_ministep_scratch_bytes": (c_size_t, [POINTER(c_ministep_args)]),
    "db_ministep_lookahead": (None, [P, P, P, P, c_size_t]),
    "db_ministep": (None, [POINTER(c_ministep_args)]),
    "db_batch_bytes": (c_size_t, [c_uint32, c_size_t, c_uint32, c_int]),
    "db_build_batch": (None, [P, P, c_uint32, c_uint32, c_int, P, P]),
    "db_build_windows": (None, [P, P, P, c_uint32, c_uint32, c_uint32, c_uint32, c_uint32, c_int, P, P]),
    "db_scanpool_fwd": (None, [P, c_uint32, c_uint32, P, c_int, P, c_uint32, P, c_uint32, c_int, P, P, P]),
    "db_scanpool_bwd": (None, [c_uint32, c_uint32, P, c_uint32, P, c_uint32, c_int, P, P, P, P, P]),
    "db_tc_weights_bytes": (c_size_t, [c_uint32, c_uint32, c_int]),
    "db_tc_prepare": (None, [P, c_uint32, c_uint32, c_int, P]),
    "db_scanpool_tc_debug": (None, [c_uint64, c_int]),
    "db_scanpool_tc_peers": (None, [c_void_p, c_uint32, c_uint32]),
    "db_scanpool_tc": (None, [P, c_uint32, c_uint32, c_int, P, c_int, P, c_uint32, P, c_uint32, c_int,
                              P, P, P, c_uint32, P, P]),
}

_NO_ERROR_CHECK = {"api_get_last_error", "api_clear_last_error", "api_device_count", "api_get_stream", "api_launch_count", "db_scratch_bytes",
                   "db_ministep_supported", "db_ministep_scratch_bytes"}


class _SafeFunc(object):
    def __init__(self, name, func, dll):
        self._name, self._func, self._dll = name, func, dll

    def __call__(self, *args):
        rval = self._func(*args)
        msg = self._dll.api_get_last_error()
        if msg is None:
            return rval
        self._dll.api_clear_last_error()
        raise SmatException("%s(...) raised an exception\n%s" % (self._name.replace("api_", ""), msg.decode()))


class _SafeDll(object):
    def __init__(self, dll):
        self._dll = dll
        for name, (restype, argtypes) in _PROTOTYPES.items():
            f = getattr(dll, name)      # AttributeError here means the .so is stale
            f.restype, f.argtypes = restype, argtypes
            setattr(self, name, f if name in _NO_ERROR_CHECK else _SafeFunc(name, f, dll))


_dll = None


def exported_names():
    return sorted(_PROTOTYPES)


def load():
    """Loads the native library or raises; never substitutes another backend."""
    global _dll
    if _dll is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("deepbind_b200: %s is missing. Build it with `python -m deepbind_b200.build` "
                              "(needs nvcc); there is no CPU or PyTorch fallback." % LIB_PATH)
        _dll = _SafeDll(ctypes.CDLL(LIB_PATH))
    return _dll
