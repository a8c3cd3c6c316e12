"""Bit packers and operator lookup with the reference's names and semantics.

Mirror of the reference's ``src/nanoquant/kernel/utils.py`` for the inference
path: the same functions, arguments, return values and error behaviour, but
every function runs a CUDA kernel of ``libnanoquant_b200.so`` through the C ABI
instead of chains of PyTorch elementwise ops.  Outputs are bit-identical to the
reference's (pinned by ``tests/golden``).

Tensors may live on a CUDA device or on the CPU; CPU tensors are staged through
the current CUDA device (the kernels are the only implementation: without a
CUDA device these functions raise).
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import _lib

MARLIN_MIN_MAX_PAR = 32  # reference: src/nanoquant/kernel/utils.py:21


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _to_cuda(t: torch.Tensor) -> torch.Tensor:
    if t.is_cuda:
        return t.contiguous()
    if not torch.cuda.is_available():
        raise RuntimeError("nanoquant_b200 packers need a CUDA device: there is no CPU implementation")
    return t.contiguous().cuda()


def _check_method(method: str) -> int:
    if method not in _lib.ORDER_ID:
        raise ValueError(f"Unsupported method: '{method}'. Supported methods are 'lsb_first', 'half2'.")
    return _lib.ORDER_ID[method]


def get_kernel_function(namespace: str, dtype: torch.dtype, kernel_type: str):
    """Reference ``get_kernel_function`` (``kernel/utils.py:33-48``): returns
    ``torch.ops.binary_kernels.<namespace>[_dyn]_forward``."""
    try:
        import binary_kernels  # noqa: F401  registers the operators
    except Exception as exc:
        raise ImportError("Could not import `binary_kernels`. Did you build the extension?\n"
                          f"Original error: {exc}") from exc
    mid = "_dyn" if kernel_type != "fixed" else ""
    op_name = f"{namespace}{mid}_forward"
    try:
        return getattr(torch.ops.binary_kernels, op_name)
    except AttributeError as exc:
        have = dir(torch.ops.binary_kernels) if hasattr(torch.ops, "binary_kernels") else []
        raise AttributeError(f"Dispatcher op `{namespace}::{op_name}` not found. "
                             f"Available in torch.ops.binary_kernels: {have}") from exc


def pack_binary_gemv(tensor: torch.Tensor, method: str = "lsb_first") -> torch.Tensor:
    """±1 int8 ``(rows, cols)`` -> int32 ``(rows, ceil(cols/32))``; reference
    ``pack_binary_gemv`` (``kernel/utils.py:51-113``)."""
    if tensor.dtype != torch.int8:
        raise TypeError("Input tensor must be int8.")
    order = _check_method(method)
    rows, cols = tensor.shape
    src = _to_cuda(tensor)
    out = torch.empty((rows, (cols + 31) // 32), dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_pack_rows(src.data_ptr(), out.data_ptr(), rows, cols, order,
                                           _stream(src.device)), "nq_pack_rows")
    return out.to(tensor.device)


def unpack_binary_gemv(packed_tensor: torch.Tensor, original_shape: Tuple[int, int],
                       method: str = "lsb_first") -> torch.Tensor:
    """Inverse of :func:`pack_binary_gemv`; reference ``unpack_binary_gemv``
    (``kernel/utils.py:116-183``)."""
    if packed_tensor.dim() != 2:
        raise ValueError(
            f"Unsupported packed tensor format. Expected 2D tensor, got {packed_tensor.dim()} dimensions.")
    rows, cols = int(original_shape[0]), int(original_shape[1])
    words = (cols + 31) // 32
    if tuple(packed_tensor.shape) != (rows, words):
        raise ValueError(
            f"Unsupported packed tensor shape. Expected ({rows}, {words}), got {packed_tensor.shape}.")
    order = _check_method(method)
    src = _to_cuda(packed_tensor.to(torch.int32))
    out = torch.empty((rows, cols), dtype=torch.int8, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_unpack_rows(src.data_ptr(), out.data_ptr(), rows, cols, order,
                                             _stream(src.device)), "nq_unpack_rows")
    return out.to(packed_tensor.device)


def reorder_packed(packed: torch.Tensor, method_in: str, method_out: str) -> torch.Tensor:
    """Change the bit order of packed words (e.g. checkpoint ``lsb_first`` ->
    ``half2``) without the dense detour of the reference loader."""
    src = _to_cuda(packed)
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_reorder_words(src.data_ptr(), out.data_ptr(), src.numel(),
                                               _check_method(method_in), _check_method(method_out),
                                               _stream(src.device)), "nq_reorder_words")
    return out.to(packed.device)


def _permute_scale(s: torch.Tensor, kind: int, inverse: bool = False) -> torch.Tensor:
    group = 16 if kind == 0 else 32
    if s.numel() % group:
        raise RuntimeError(f"scale of {s.numel()} elements is not a multiple of {group}")
    if s.element_size() != 2:
        raise TypeError("scale vectors must be fp16 or bf16 (the dtypes the kernels compute in)")
    src = _to_cuda(s.reshape(-1))
    out = torch.empty_like(src)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_permute_scale16(src.data_ptr(), out.data_ptr(), src.numel(), kind,
                                                 int(inverse), _stream(src.device)), "nq_permute_scale16")
    return out.to(s.device)


def pack_binary_marlin(weight: torch.Tensor, scale_in: torch.Tensor, scale_out: torch.Tensor):
    """``weight [out, in]`` ±1 -> ``(B [in/16, out/2] int32, scale_in', scale_out',
    workspace_size)``; reference ``pack_binary_marlin`` (``kernel/utils.py:186-214``)."""
    out_f, in_f = weight.shape
    if out_f % 64 or in_f % 16:
        raise RuntimeError(f"shape '[{out_f // 64}, 4, 2, 8, {in_f // 16}, 2, 4, 2]' is invalid for input of size "
                           f"{out_f * in_f}")
    src = _to_cuda(weight.to(torch.int8))
    B = torch.empty((in_f // 16, out_f // 2), dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_pack_marlin(src.data_ptr(), B.data_ptr(), out_f, in_f,
                                             _stream(src.device)), "nq_pack_marlin")
    s_in = _permute_scale(scale_in, 0)
    s_out = _permute_scale(scale_out, 1)
    workspace_size = s_out.numel() // 128 * MARLIN_MIN_MAX_PAR
    return B.to(weight.device), s_in, s_out, workspace_size


def pack_binary_marlin_fused(V_sign: torch.Tensor, U_sign: torch.Tensor, scale_g: torch.Tensor,
                             scale_l: torch.Tensor, scale_h: torch.Tensor):
    """Two-stage Marlin packing with the rank padded to a multiple of 256 (+1
    signs, zero ``scale_l``); reference ``pack_binary_marlin_fused``
    (``kernel/utils.py:217-284``).  ``V_sign`` is ``[N, R]``, ``U_sign`` ``[R, M]``."""
    dev = V_sign.device
    N = scale_g.shape[0]
    R = scale_l.shape[0] if scale_l is not None else U_sign.shape[0]
    M = scale_h.shape[0]
    N, R, M = [(d + 31) // 32 * 32 for d in (N, R, M)]
    rank_marlin = (R + 255) // 256 * 256
    if rank_marlin > R:
        pad = rank_marlin - R
        V_sign = torch.cat([V_sign, torch.ones(N, pad, device=dev, dtype=torch.int8)], dim=1)
        U_sign = torch.cat([U_sign, torch.ones(pad, M, device=dev, dtype=torch.int8)], dim=0)
        if scale_l is not None:
            scale_l = torch.cat([scale_l, torch.zeros(pad, device=dev, dtype=scale_l.dtype)], dim=0)
    V_bits, s_g, s_l, ws_v = pack_binary_marlin(V_sign.T, scale_g, scale_l)
    U_bits, _, s_h, ws_u = pack_binary_marlin(U_sign.T, scale_l, scale_h)
    workspace = torch.zeros(max(ws_v, ws_u), device=dev, dtype=torch.int32)
    return V_bits.contiguous(), U_bits.contiguous(), s_g, s_l, s_h, workspace


# --- runtime tile layout of the GEMV kernel ----------------------------------

def tiles_shape(rows: int, cols: int) -> Tuple[int, int, int]:
    return ((rows + 15) // 16, (cols + 255) // 256, 128)


def pack_tiles(packed: torch.Tensor, shape: Tuple[int, int], method: str = "lsb_first") -> torch.Tensor:
    """rows layout ``(rows, ceil(cols/32))`` -> int32 ``(ceil(rows/16), ceil(cols/256), 128)``
    tile layout consumed by the GEMV kernel (``nq_rows_to_tiles``)."""
    rows, cols = int(shape[0]), int(shape[1])
    if tuple(packed.shape) != (rows, (cols + 31) // 32):
        raise ValueError(f"packed tensor of shape {tuple(packed.shape)} does not hold a {rows}x{cols} matrix")
    src = _to_cuda(packed.to(torch.int32))
    out = torch.empty(tiles_shape(rows, cols), dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_rows_to_tiles(src.data_ptr(), out.data_ptr(), rows, cols, _check_method(method),
                                               _stream(src.device)), "nq_rows_to_tiles")
    out._nq_rows, out._nq_cols = rows, cols   # exact shape: the tiles pad rows to 16 and columns to 256
    return out


def unpack_tiles(tiles: torch.Tensor, shape: Tuple[int, int], method: str = "lsb_first") -> torch.Tensor:
    """Inverse of :func:`pack_tiles`."""
    rows, cols = int(shape[0]), int(shape[1])
    if tuple(tiles.shape) != tiles_shape(rows, cols):
        raise ValueError(f"tile tensor of shape {tuple(tiles.shape)} does not hold a {rows}x{cols} matrix")
    src = _to_cuda(tiles)
    out = torch.empty((rows, (cols + 31) // 32), dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().nq_tiles_to_rows(src.data_ptr(), out.data_ptr(), rows, cols, _check_method(method),
                                               _stream(src.device)), "nq_tiles_to_rows")
    return out


# reference aliases (kernel/utils.py:503-507)
binary_packer = pack_binary_gemv
binary_unpacker = unpack_binary_gemv
marlin_onebit_packer = pack_binary_marlin
marlin_nanoquant_packer = pack_binary_marlin_fused
