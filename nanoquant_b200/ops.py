"""``torch.ops.binary_kernels.*`` — the reference's dispatcher operators, backed
by ``libnanoquant_b200.so``.

The three schemas are the reference's, verbatim
(``src/nanoquant/kernel/pybind.cpp:83-105``); CUDA implementations call the C
ABI with ``data_ptr()`` and the current stream, fake (Meta) implementations
give shapes for tracing (``pybind.cpp:11-31``, ``cuda/gemm.cpp:100-134``).
Nothing here computes on the CPU.

Operand layouts accepted by ``nanoquant_dyn_forward``:

* 2-D int32 ``[rows, cols/32]`` in ``half2`` bit order — what the reference's
  ``binary_packer(..., method="half2")`` produces.  Converted once to the tile
  layout of the kernel and cached on the tensor object.
* 3-D int32 ``[rows/16, ceil(cols/256), 128]`` — the tile layout itself
  (``nanoquant_b200.kernel.utils.pack_tiles``), used as is.

Note the reference's argument naming: ``Ubits`` is the FIRST factor (module
``V``, ``[R, N]``) and ``Vbits`` the second (module ``U``, ``[M, R]``).
"""
from __future__ import annotations

import contextlib
import ctypes
import threading
from typing import Optional

import torch

from . import _lib
from .kernel import utils as ku

_DEFINED = False

_SWEEP = {  # reference: cuda/gemv_kernel.cu:351-354
    "n_th": (64, 128, 256),
    "n_rpw": (1, 2, 4, 8),
    "n_acc": (1, 2),
    "n_pipe": (1, 2, 4, 8, 16),
}

_scratch = {}        # device index -> zero-initialised uint8 tensor
_retired = []        # outgrown scratch buffers, kept for graphs that were captured on them
_SCRATCH_MIN = 4 << 20
_override = threading.local()   # .buf: a caller-provided scratch for this thread (see private_scratch)


def _check_sweep(name: str, kind: str, value: int) -> None:
    """The reference dispatches the tuning arguments through compile-time
    lists and raises ``ValueError`` on a miss (``cuda/meta_utils.h:14-38``).  The
    kernel here has no such knobs; the values are validated the same way and
    otherwise ignored."""
    choices = _SWEEP[kind]
    if value not in choices:
        raise ValueError(f"{name} should be one of [{', '.join(map(str, choices))}], but {value} was given")


def reserve_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Make sure the scratch of `device` holds `nbytes` (called when a layer is prepared, i.e. before any forward
    and outside any stream capture or graph memory pool): the buffer is allocated once, for the device's largest
    layer, and every later launch only reads its address."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    buf = _scratch.get(idx)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("nanoquant_b200: the kernels' scratch buffer would have to be (re)allocated inside a "
                               "stream capture; prepare the layers (or call nanoquant_b200.ops.reserve_scratch) first")
        if buf is not None:
            _retired.append(buf)   # a CUDA graph captured earlier may still point at the smaller buffer: keep it alive
        buf = torch.zeros(max(int(nbytes), _SCRATCH_MIN), dtype=torch.uint8, device=torch.device("cuda", idx))
        _scratch[idx] = buf
    return buf


def set_precise_intermediate(on: bool) -> bool:
    """bf16 linears through the GEMM path (5 tokens and more): keep the rank-R intermediate as fp16 times a
    per-token power of two instead of rounding it to bf16 between the stages (one more small kernel per launch
    group; see ``nq_gemm_set_precise_intermediate``).  Process-wide; returns the previous setting."""
    return bool(_lib.lib().nq_gemm_set_precise_intermediate(1 if on else 0))


def group_scratch_bytes(shapes, T: int) -> int:
    """Scratch bytes one launch group of linears with ``shapes = [(N, R, M), ...]`` needs at `T` tokens."""
    L = _lib.lib()
    arr = (_lib.LinearDesc * len(shapes))()
    for d, (N, R, M) in zip(arr, shapes):
        d.N, d.R, d.M = int(N), int(R), int(M)
    if T <= L.nq_gemv_max_tokens():
        return int(L.nq_gemv_group_scratch_bytes(arr, len(shapes), T))
    return int(L.nq_gemm_group_scratch_bytes(arr, len(shapes), T))


def scratch_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """The scratch the kernels of `device` run on: one buffer per device, zeroed once at allocation as the C ABI
    asks.  Launches that share it must be ordered on one stream (what a model forward and its graph capture
    are); code that runs layers on several streams at once gives each stream its own buffer with
    :func:`private_scratch`."""
    buf = getattr(_override, "buf", None)
    if buf is not None:
        if buf.numel() < nbytes:
            raise RuntimeError(f"private scratch of {buf.numel()} bytes is too small: {nbytes} needed")
        return buf
    return reserve_scratch(device, nbytes)


@contextlib.contextmanager
def private_scratch(buf: torch.Tensor):
    """Run the enclosed launches of this thread on `buf` (uint8, zeroed once by the caller, 16-byte aligned)
    instead of the device's shared scratch: for concurrent streams."""
    prev = getattr(_override, "buf", None)
    _override.buf = buf
    try:
        yield buf
    finally:
        _override.buf = prev


def _dtype_id(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return _lib.NQ_F16
    if t.dtype == torch.bfloat16:
        return _lib.NQ_BF16
    raise RuntimeError("Support only Half or BFloat16")


def _check_cuda_cont(t: torch.Tensor, name: str, dtype: torch.dtype, dtype_name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype_name} tensor")


def as_tiles(bits: torch.Tensor, cols: int) -> torch.Tensor:
    """Tile-layout view of a factor given in either accepted layout."""
    if bits.dim() == 3:
        return bits
    cached = getattr(bits, "_nq_tiles", None)
    if cached is not None and cached[0] == bits._version:
        return cached[1]
    rows = bits.size(0)
    if bits.size(1) != (cols + 31) // 32:
        raise RuntimeError(f"packed factor of shape {tuple(bits.shape)} does not match {cols} columns")
    tiles = ku.pack_tiles(bits, (rows, cols), method="half2")
    bits._nq_tiles = (bits._version, tiles)
    return tiles


def gemv_forward(x: torch.Tensor, s_in: torch.Tensor, v_tiles: torch.Tensor, s_mid: Optional[torch.Tensor],
                 u_tiles: torch.Tensor, s_out: torch.Tensor, R: int) -> torch.Tensor:
    """Launch ``nq_gemv_fwd`` on the current stream; ``x`` is ``[T, N]``."""
    T, N = x.shape
    M = s_out.size(0)
    y = torch.empty((T, M), dtype=x.dtype, device=x.device)
    if T == 0:
        return y
    L = _lib.lib()
    nbytes = L.nq_gemv_scratch_bytes(T, N, R, M)
    scratch = scratch_for(x.device, nbytes)
    with torch.cuda.device(x.device):
        st = L.nq_gemv_fwd(x.data_ptr(), s_in.data_ptr(), v_tiles.data_ptr(),
                           s_mid.data_ptr() if s_mid is not None else None,
                           u_tiles.data_ptr(), s_out.data_ptr(), y.data_ptr(),
                           scratch.data_ptr(), scratch.numel(), T, N, R, M, _dtype_id(x),
                           torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(st, "nq_gemv_fwd")
    return y


def dense_gemv_forward(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.linear(x, weight, bias)`` for the few tokens of a decode step through ``nq_dense_gemv_fwd``.

    For the layers the reference leaves as ``nn.Linear`` (``lm_head``, ``utils/load_utils.py:322``): ``weight``
    ``[V, N]`` fp16/bf16 with a unit inner stride, ``x`` ``[..., N]`` with at most ``nq_dense_gemv_max_tokens()``
    rows in total; more rows raise (a batched GEMM is the right tool there)."""
    _check_cuda_cont(x, "x", weight.dtype, str(weight.dtype))
    if weight.dim() != 2 or weight.stride(1) != 1 or not weight.is_cuda:
        raise RuntimeError("weight must be a CUDA [V, N] matrix with a unit inner stride")
    if x.size(-1) != weight.size(1):
        raise RuntimeError(f"x has {x.size(-1)} columns, weight expects {weight.size(1)}")
    if bias is not None:
        _check_cuda_cont(bias, "bias", weight.dtype, str(weight.dtype))
    V, N = weight.shape
    x2 = x.reshape(-1, N)
    T = x2.size(0)
    y = torch.empty((T, V), dtype=x.dtype, device=x.device)
    if T > 0:
        L = _lib.lib()
        with torch.cuda.device(x.device):
            st = L.nq_dense_gemv_fwd(x2.data_ptr(), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                                     y.data_ptr(), T, N, V, weight.stride(0), V, _dtype_id(x),
                                     torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(st, "nq_dense_gemv_fwd")
    return y.reshape(*x.shape[:-1], V)


def _nanoquant_dyn_forward_cuda(x, scale_g, Ubits, scale_l, Vbits, scale_h,
                                num_thread_stage1=128, num_thread_stage2=128,
                                num_row_per_warp_stage1=2, num_row_per_warp_stage2=2,
                                num_acc_stage1=4, num_acc_stage2=4,
                                num_pipeline_stage1=2, num_pipeline_stage2=2):
    # checks in the order of the reference host function (cuda/gemv_kernel.cu:317-338)
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("Support only Half or BFloat16")
    name = "float16" if x.dtype == torch.float16 else "bfloat16"
    _check_cuda_cont(x, "x", x.dtype, name)
    _check_cuda_cont(scale_g, "scale_g", x.dtype, name)
    _check_cuda_cont(scale_h, "scale_h", x.dtype, name)
    _check_cuda_cont(Ubits, "Ubits", torch.int32, "int32")
    _check_cuda_cont(Vbits, "Vbits", torch.int32, "int32")
    N = x.size(-1)
    M = scale_h.size(0)
    if Ubits.dim() == 3:
        # the tile tensor covers ceil(R / 16) * 16 rows; the exact rank comes from scale_l or from the packer's note
        R = scale_l.size(0) if scale_l is not None else getattr(Ubits, "_nq_rows", None)
        if R is None:
            if Vbits.dim() == 3 and hasattr(Vbits, "_nq_cols"):
                R = Vbits._nq_cols
            else:
                raise RuntimeError("rank of tile-layout operands unknown: pass scale_l, or tiles made by "
                                   "nanoquant_b200.kernel.utils.pack_tiles (which records the matrix shape)")
    else:
        R = Ubits.size(0)
    if scale_l is not None:
        _check_cuda_cont(scale_l, "(*scale_l)", x.dtype, name)
        if scale_l.size(0) != R:
            raise RuntimeError("scale_l size mismatch")
    if scale_g.size(0) != N:
        raise RuntimeError("scale_g size mismatch")
    _check_sweep("n_th1", "n_th", num_thread_stage1)
    _check_sweep("n_rpw1", "n_rpw", num_row_per_warp_stage1)
    _check_sweep("n_acc1", "n_acc", num_acc_stage1)
    _check_sweep("n_pipe1", "n_pipe", num_pipeline_stage1)
    _check_sweep("n_th2", "n_th", num_thread_stage2)
    _check_sweep("n_rpw2", "n_rpw", num_row_per_warp_stage2)
    _check_sweep("n_acc2", "n_acc", num_acc_stage2)
    _check_sweep("n_pipe2", "n_pipe", num_pipeline_stage2)
    v_tiles = as_tiles(Ubits, N)
    u_tiles = as_tiles(Vbits, R)
    x2 = x.view(1, N) if x.dim() == 1 else x
    y = linear_forward(x2, scale_g, v_tiles, scale_l, u_tiles, scale_h, R)
    return y.squeeze(0) if x.dim() == 1 else y


def _nanoquant_dyn_forward_fake(x, scale_g, Ubits, scale_l, Vbits, scale_h, *args, **kwargs):
    shape = list(x.shape)
    shape[-1] = scale_h.size(0)
    return x.new_empty(shape)


def group_forward(xs, layers, T: int, dtype: torch.dtype, device: torch.device, biases=None, residuals=None,
                  out: Optional[torch.Tensor] = None):
    """One launch group: up to four linears in one ``nq_gemv_group_fwd`` (T <= 4) or ``nq_gemm_group_fwd`` call.

    ``xs[i]`` ``[T, N_i]`` (row stride free, unit inner stride), ``layers[i] = (s_in, v_tiles, s_mid, u_tiles, s_out, R)``,
    optional ``biases[i]`` ``[M_i]`` and ``residuals[i]`` ``[T, M_i]`` (added in fp32 behind the output scale).  The
    outputs are written side by side into one ``[T, sum(M_i)]`` buffer (``out`` or a fresh one); returns its
    per-linear column views."""
    n = len(layers)
    Ms = [lay[4].size(0) for lay in layers]
    width = sum(Ms)
    if out is None:
        out = torch.empty((T, width), dtype=dtype, device=device)
    views, col = [], 0
    for m in Ms:
        views.append(out[:, col:col + m])
        col += m
    if T == 0:
        return views
    L = _lib.lib()
    descs, col = [], 0
    for i, (s_in, v_tiles, s_mid, u_tiles, s_out, R) in enumerate(layers):
        x = xs[i]
        if x.stride(-1) != 1:
            raise RuntimeError("group_forward: activations need a unit inner stride")
        b = biases[i] if biases is not None else None
        r = residuals[i] if residuals is not None else None
        if r is not None and r.stride(-1) != 1:
            raise RuntimeError("group_forward: residual needs a unit inner stride")
        descs.append(_lib.LinearDesc(
            x.data_ptr(), s_in.data_ptr(), v_tiles.data_ptr(), s_mid.data_ptr() if s_mid is not None else None,
            u_tiles.data_ptr(), s_out.data_ptr(), out.data_ptr() + col * out.element_size(),
            x.size(-1), R, Ms[i], x.stride(0) if x.dim() == 2 else x.size(-1), out.stride(0),
            b.data_ptr() if b is not None else None, r.data_ptr() if r is not None else None,
            r.stride(0) if r is not None else 0))
        col += Ms[i]
    arr = (_lib.LinearDesc * n)(*descs)
    gemv = T <= L.nq_gemv_max_tokens()
    size_fn, fwd = ((L.nq_gemv_group_scratch_bytes, L.nq_gemv_group_fwd) if gemv
                    else (L.nq_gemm_group_scratch_bytes, L.nq_gemm_group_fwd))
    scratch = scratch_for(device, size_fn(arr, n, T))
    with torch.cuda.device(device):
        st = fwd(arr, n, T, _dtype_id(out), scratch.data_ptr(), scratch.numel(),
                 torch.cuda.current_stream(device).cuda_stream)
    _lib.check(st, "nq_gemv_group_fwd" if gemv else "nq_gemm_group_fwd")
    return views


def linear_forward(x: torch.Tensor, s_in: torch.Tensor, v_tiles: torch.Tensor, s_mid: Optional[torch.Tensor],
                   u_tiles: torch.Tensor, s_out: torch.Tensor, R: int, bias: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``nq_linear_fwd``: GEMV for few tokens, tcgen05 GEMM above; ``x`` is ``[T, N]``.  With ``bias`` / ``residual``
    the call goes through the group entry points, whose descriptors carry them into the kernels' epilogues."""
    T, N = x.shape
    M = s_out.size(0)
    if bias is not None or residual is not None:
        return group_forward([x], [(s_in, v_tiles, s_mid, u_tiles, s_out, R)], T, x.dtype, x.device,
                             [bias], [residual])[0]
    y = torch.empty((T, M), dtype=x.dtype, device=x.device)
    if T == 0:
        return y
    L = _lib.lib()
    scratch = scratch_for(x.device, L.nq_linear_scratch_bytes(T, N, R, M))
    with torch.cuda.device(x.device):
        st = L.nq_linear_fwd(x.data_ptr(), s_in.data_ptr(), v_tiles.data_ptr(),
                             s_mid.data_ptr() if s_mid is not None else None,
                             u_tiles.data_ptr(), s_out.data_ptr(), y.data_ptr(),
                             scratch.data_ptr(), scratch.numel(), T, N, R, M, _dtype_id(x),
                             torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(st, "nq_linear_fwd")
    return y


# --- Marlin-layout operands -----------------------------------------------------------------

def _marlin_as_tiles(B: torch.Tensor) -> torch.Tensor:
    """Marlin-fragment words ``[in/16, out/2]`` (what the reference's ``pack_binary_marlin``
    produces) -> tile layout of the kernels here, cached on the tensor object."""
    cached = getattr(B, "_nq_tiles", None)
    if cached is not None and cached[0] == B._version:
        return cached[1]
    in_f, out_f = B.size(0) * 16, B.size(1) * 2
    if in_f % 32 or out_f % 64:
        raise RuntimeError("Problem shape incompatible")
    L = _lib.lib()
    rows = torch.empty((out_f, in_f // 32), dtype=torch.int32, device=B.device)
    with torch.cuda.device(B.device):
        _lib.check(L.nq_marlin_to_rows(B.data_ptr(), rows.data_ptr(), out_f, in_f, _lib.NQ_LSB_FIRST,
                                       torch.cuda.current_stream(B.device).cuda_stream), "nq_marlin_to_rows")
    tiles = ku.pack_tiles(rows, (out_f, in_f), "lsb_first")
    B._nq_tiles = (B._version, tiles)
    return tiles


def _unpermuted_scale(s: Optional[torch.Tensor], kind: int) -> Optional[torch.Tensor]:
    """Undo the Marlin scale permutation (cached on the tensor object)."""
    if s is None:
        return None
    cached = getattr(s, "_nq_plain", None)
    if cached is not None and cached[0] == s._version:
        return cached[1]
    plain = ku._permute_scale(s.contiguous(), kind, inverse=True)
    s._nq_plain = (s._version, plain)
    return plain


MARLIN_MIN_MAX_PAR = 32  # reference: src/nanoquant/kernel/cuda/gemm.cpp:33


def _marlin_checks(A, B, s_in, s_out, workspace):
    # reference: marlin_onebit_check_and_alloc, src/nanoquant/kernel/cuda/gemm.cpp:36-56
    prob_n, prob_k = B.size(1) * 2, A.size(1)
    if prob_k != B.size(0) * 16:
        raise RuntimeError("k dimension mismatch")
    if s_in is not None and s_in.size(0) != prob_k:
        raise RuntimeError("s_in size mismatch")
    if s_out is not None and s_out.size(0) != prob_n:
        raise RuntimeError("s_out size mismatch")
    if workspace.numel() < prob_n // 128 * MARLIN_MIN_MAX_PAR:
        raise RuntimeError("workspace too small")
    if A.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("Unsupported dtype: Marlin only supports Half and BFloat16")
    return prob_n, prob_k


def _status_words(device: torch.device) -> torch.Tensor:
    return scratch_for(device, 256)


def _marlin_onebit_forward_cuda(x, weight, scale_g, scale_h, workspace):
    prob_n, prob_k = _marlin_checks(x, weight, scale_g, scale_h, workspace)
    x = x.contiguous()
    tiles = _marlin_as_tiles(weight)
    s_in = _unpermuted_scale(scale_g, 0)
    s_out = _unpermuted_scale(scale_h, 1)
    T = x.size(0)
    y = torch.empty((T, prob_n), dtype=x.dtype, device=x.device)
    if T == 0:
        return y
    L = _lib.lib()
    with torch.cuda.device(x.device):
        st = L.nq_onebit_gemm_fwd(x.data_ptr(), tiles.data_ptr(),
                                  s_in.data_ptr() if s_in is not None else None,
                                  s_out.data_ptr() if s_out is not None else None,
                                  y.data_ptr(), _status_words(x.device).data_ptr(), T, prob_k, prob_n,
                                  _dtype_id(x), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(st, "nq_onebit_gemm_fwd")
    return y


def _marlin_onebit_forward_fake(x, weight, scale_g, scale_h, workspace):
    return x.new_empty((x.size(0), weight.size(1) * 2))


def _marlin_nanoquant_forward_cuda(x, weight_u, weight_v, scale_g, scale_l, scale_h, workspace):
    # `weight_u` is the FIRST stage (module V), `weight_v` the second (reference gemm.cpp:112-122)
    if weight_u.dim() == 3:
        # operands already in the kernels' tile layout, scales in plain order (what this package's own module
        # keeps for kernel_type="gemm": one copy of the weights instead of Marlin words plus converted tiles)
        if scale_g is None or scale_h is None:
            raise RuntimeError("scale_g and scale_h are required")
        R = scale_l.size(0) if scale_l is not None else getattr(weight_u, "_nq_rows", weight_u.size(0) * 16)
        return linear_forward(x.contiguous(), scale_g, weight_u, scale_l, weight_v, scale_h, R)
    R, N = _marlin_checks(x, weight_u, scale_g, scale_l, workspace)
    if scale_g is None or scale_h is None:
        raise RuntimeError("scale_g and scale_h are required")
    M = weight_v.size(1) * 2
    if weight_v.size(0) * 16 != R:
        raise RuntimeError("k dimension mismatch")
    if scale_h.size(0) != M:
        raise RuntimeError("s_out size mismatch")
    if workspace.numel() < M // 128 * MARLIN_MIN_MAX_PAR:
        raise RuntimeError("workspace too small")
    x = x.contiguous()
    return linear_forward(x, _unpermuted_scale(scale_g, 0), _marlin_as_tiles(weight_u),
                          _unpermuted_scale(scale_l, 1), _marlin_as_tiles(weight_v),
                          _unpermuted_scale(scale_h, 1), R)


def _marlin_nanoquant_forward_fake(x, weight_u, weight_v, scale_g, scale_l, scale_h, workspace):
    return x.new_empty((x.size(0), weight_v.size(1) * 2))


def define_ops() -> None:
    """Define and register the operators once per process."""
    global _DEFINED
    if _DEFINED:
        return
    torch.library.define(
        "binary_kernels::nanoquant_dyn_forward",
        "(Tensor x, Tensor scale_g, Tensor Ubits, Tensor? scale_l, Tensor Vbits, Tensor scale_h, "
        "int num_thread_stage1=128, int num_thread_stage2=128, int num_row_per_warp_stage1=2, "
        "int num_row_per_warp_stage2=2, int num_acc_stage1=4, int num_acc_stage2=4, "
        "int num_pipeline_stage1=2, int num_pipeline_stage2=2) -> Tensor")
    torch.library.impl("binary_kernels::nanoquant_dyn_forward", "CUDA")(_nanoquant_dyn_forward_cuda)
    torch.library.register_fake("binary_kernels::nanoquant_dyn_forward")(_nanoquant_dyn_forward_fake)
    torch.library.define(
        "binary_kernels::marlin_onebit_forward",
        "(Tensor x, Tensor weight, Tensor? scale_g, Tensor? scale_h, Tensor(a!) workspace) -> Tensor")
    torch.library.impl("binary_kernels::marlin_onebit_forward", "CUDA")(_marlin_onebit_forward_cuda)
    torch.library.register_fake("binary_kernels::marlin_onebit_forward")(_marlin_onebit_forward_fake)
    torch.library.define(
        "binary_kernels::marlin_nanoquant_forward",
        "(Tensor x, Tensor weight_u, Tensor weight_v, Tensor? scale_g, Tensor? scale_l, Tensor? scale_h, "
        "Tensor(a!) workspace) -> Tensor")
    torch.library.impl("binary_kernels::marlin_nanoquant_forward", "CUDA")(_marlin_nanoquant_forward_cuda)
    torch.library.register_fake("binary_kernels::marlin_nanoquant_forward")(_marlin_nanoquant_forward_fake)
    _DEFINED = True
