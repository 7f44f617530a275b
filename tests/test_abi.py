"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and refuses to compute without a device (no CPU fallback)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    src = open(os.path.join(ROOT, "include", "deepbind_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", src)
    return sorted({n for n in names if n.startswith(("api_", "db_", "register_ext"))})


def test_every_declared_symbol_is_exported():
    from deepbind_b200 import _lib
    assert os.path.exists(_lib.LIB_PATH), "build the library first: python -m deepbind_b200.build"
    dll = ctypes.CDLL(_lib.LIB_PATH)
    declared = header_functions()
    assert len(declared) >= 50
    missing = [n for n in declared if not hasattr(dll, n)]
    assert not missing, missing


def test_python_prototypes_cover_the_header():
    from deepbind_b200 import _lib
    assert set(header_functions()) == set(_lib.exported_names())


def test_reference_entry_point_names_are_present():
    # kangaroo_smat.cpp:333-418 and deepity_smat.cpp:497-607
    want = """api_corr1ord api_corr1ord_bprop_W api_corr1ord_bprop_X api_poolrgn api_poolrgn_bprop
              api_dropoutord_fp_tr api_autotune register_ext api_gradstep api_gradstep_nesterov1
              api_gradstep_nesterov2 api_madd_bcast api_maskout api_calc_zmask api_dropout_fp_tr
              api_dropout_fp_te api_dropout_bp_tr api_dropout_bp_te api_blockwise_dot api_blockwise_dot_nt
              api_blockwise_dot_tn api_blockwise_dot_combined api_blockwise_dot_nt_combined
              api_blockwise_dot_tn_combined api_get_last_error api_clear_last_error api_sync""".split()
    from deepbind_b200 import _lib
    dll = ctypes.CDLL(_lib.LIB_PATH)
    for n in want:
        assert hasattr(dll, n), n


def test_option_struct_layouts():
    from deepbind_b200 import _lib
    assert ctypes.sizeof(_lib.c_corr1ord_options_t) == 8       # {int padmode; uint32 nchannel}
    assert ctypes.sizeof(_lib.c_poolrgn_options_t) == 4        # {int ptype}
    assert _lib.c_corr1ord_options_t.nchannel.offset == 4


def test_ministep_args_layout_matches_the_header(tmp_path):
    """ctypes mirror of struct db_ministep_args against the C compiler's layout of the header's."""
    import shutil
    import subprocess
    from deepbind_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    names = [n for n, _ in _lib.c_ministep_args._fields_]
    src = tmp_path / "layout.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "deepbind_b200.h"\nint main(void) {\n'
                   '  printf("%zu\\n", sizeof(db_ministep_args));\n' +
                   "".join('  printf("%%zu\\n", offsetof(db_ministep_args, %s));\n' % n for n in names) + "  return 0;\n}\n")
    exe = tmp_path / "layout"
    inc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run([cc, "-I", inc, str(src), "-o", str(exe)], check=True)
    out = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert out[0] == ctypes.sizeof(_lib.c_ministep_args)
    assert out[1:] == [getattr(_lib.c_ministep_args, n).offset for n in names]


def test_compute_without_a_device_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from deepbind_b200 import _lib
    dll = _lib.load()
    assert dll.api_device_count() == 0
    with pytest.raises(_lib.SmatException, match="no usable CUDA device"):
        dll.db_relu(None, None, 16)
    # the error channel is cleared by the raise
    assert dll.api_get_last_error() is None


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "deepbind_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, (f, "mentions the oracle")
