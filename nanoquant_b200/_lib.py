"""ctypes binding of ``libnanoquant_b200.so`` (the C ABI in ``include/nanoquant_b200.h``).

The library is loaded from the package directory (built in-tree by
``nanoquant_b200.build``).  There is no fallback: if it is missing, loading
raises, and every operator of this package fails with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libnanoquant_b200.so")

NQ_F16, NQ_BF16 = 0, 1
NQ_LSB_FIRST, NQ_HALF2 = 0, 1
ORDER_ID = {"lsb_first": NQ_LSB_FIRST, "half2": NQ_HALF2}

NQ_OK = 0
NQ_ERR_NULL, NQ_ERR_SHAPE, NQ_ERR_DTYPE, NQ_ERR_ALIGN = -1, -2, -3, -4
NQ_ERR_SCRATCH, NQ_ERR_CUDA, NQ_ERR_TIMEOUT, NQ_ERR_UNSUPPORTED, NQ_ERR_TOO_LARGE = -5, -6, -7, -8, -9


class LinearDesc(ctypes.Structure):
    """``nq_linear_desc``."""
    _fields_ = [("x", c_void_p), ("s_in", c_void_p), ("v_tiles", c_void_p), ("s_mid", c_void_p),
                ("u_tiles", c_void_p), ("s_out", c_void_p), ("y", c_void_p),
                ("N", c_int), ("R", c_int), ("M", c_int), ("ldx", c_int64), ("ldy", c_int64),
                ("bias", c_void_p), ("residual", c_void_p), ("ldr", c_int64)]


# name -> (restype, argtypes); every symbol declared in include/nanoquant_b200.h
SIGNATURES = {
    "nq_abi_version": (c_int, []),
    "nq_strerror": (c_char_p, [c_int]),
    "nq_last_cuda_error": (c_char_p, []),
    "nq_pack_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "nq_unpack_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "nq_reorder_words": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nq_pack_marlin": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p]),
    "nq_marlin_to_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "nq_permute_scale16": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]),
    "nq_tiles_bytes": (c_size_t, [c_int64, c_int64]),
    "nq_rows_to_tiles": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "nq_tiles_to_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "nq_gemv_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nq_gemv_group_scratch_bytes": (c_size_t, [ctypes.POINTER(LinearDesc), c_int, c_int]),
    "nq_gemv_fwd": (c_int, [c_void_p] * 8 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "nq_gemv_group_fwd": (c_int, [ctypes.POINTER(LinearDesc), c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "nq_scratch_status": (c_int, [c_void_p, c_void_p]),
    "nq_gemv_set_wait_limit": (ctypes.c_uint, [ctypes.c_uint]),
    "nq_gemv_fwd_static": (c_int, [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "nq_gemv_static_max_rank": (c_size_t, []),
    "nq_gemm_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nq_gemm_set_precise_intermediate": (c_int, [c_int]),
    "nq_gemm_fwd": (c_int, [c_void_p] * 8 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "nq_gemm_group_scratch_bytes": (c_size_t, [ctypes.POINTER(LinearDesc), c_int, c_int]),
    "nq_gemm_group_fwd": (c_int, [ctypes.POINTER(LinearDesc), c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "nq_onebit_gemm_fwd": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, c_void_p]),
    "nq_allgather_state_bytes": (c_size_t, []),
    "nq_allgather_flags_bytes": (c_size_t, [c_int]),
    "nq_allgather_push": (c_int, [c_void_p, c_size_t, ctypes.POINTER(c_void_p), c_size_t, c_size_t, c_void_p, c_int, c_int,
                                  c_void_p]),
    "nq_allgather_status": (c_int, [c_void_p, c_void_p]),
    "nq_allgather_set_wait_limit": (ctypes.c_uint, [ctypes.c_uint]),
    "nq_dense_gemv_max_tokens": (c_int, []),
    "nq_dense_gemv_fwd": (c_int, [c_void_p] * 4 + [c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p]),
    "nq_gemv_max_tokens": (c_int, []),
    "nq_linear_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "nq_linear_fwd": (c_int, [c_void_p] * 8 + [c_size_t, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "nq_probe_chain": (c_int, [c_int, c_int, c_int, ctypes.POINTER(ctypes.c_float)]),
    "nq_probe_loop": (c_int, [c_int, c_int, ctypes.POINTER(ctypes.c_float)]),
}

_lib = None


class NanoQuantError(RuntimeError):
    """A C-ABI call returned a negative ``nq_status``."""

    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(what)


def lib() -> ctypes.CDLL:
    """The loaded library; raises ``ImportError`` when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found. Build it with `python -m nanoquant_b200.build` "
                "(needs nvcc); there is no CPU fallback.")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here = library older than the header
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    """Map a negative status to the exception type the reference raises for it:
    shape / dtype problems -> ``ValueError``-like ``RuntimeError`` text of the
    reference's ``TORCH_CHECK`` (``RuntimeError``), everything else likewise."""
    if status >= 0:
        return
    L = lib()
    msg = L.nq_strerror(status).decode()
    if status == NQ_ERR_CUDA:
        msg += ": " + L.nq_last_cuda_error().decode()
    raise NanoQuantError(status, f"{what}: {msg} (nq_status {status})")
