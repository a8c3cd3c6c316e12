"""nanoquant_b200 — sm_100a kernels and host API for the NanoQuant binary
low-rank quantised linear (inference path).

``libnanoquant_b200.so`` (C ABI, ``include/nanoquant_b200.h``) holds the CUDA
kernels; this package is the Python host side that mirrors the reference's
module / packer / operator interface on top of it.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
__version__ = "0.1.0"
