"""deepbind_b200: DeepBind's motif-scan / pooling / update hot path for NVIDIA B200.

The package is a thin Python mirror of the reference's extension interface over
one native library, ``lib/libdeepbind_b200.so`` (hand-written sm_100a CUDA
behind a C ABI, see ``include/deepbind_b200.h``).  Build it in-tree with
``python -m deepbind_b200.build``.  There is no CPU or PyTorch fallback.
"""
from ._lib import SmatException, LIB_PATH  # noqa: F401

__all__ = ["SmatException", "LIB_PATH"]
