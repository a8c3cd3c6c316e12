"""``NanoQuantLinear`` — the quantised linear module, inference side.

Same attribute names, state-dict keys and call protocol as the reference's
``src/nanoquant/modules/linear.py`` so that the reference's loader
(class-swap of ``nn.Linear`` + ``init_for_inference`` + ``load_state_dict``,
``src/nanoquant/utils/load_utils.py:319-335``) and its decode benchmark
(``_prepare_kernel`` on every module, ``src/nanoquant/kernel/test_decode.py:1228-1234``)
work unchanged.  Only the kernel inference path exists here: ``forward`` before
``_prepare_kernel`` raises instead of running dense PyTorch matmuls.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..kernel.utils import binary_packer, get_kernel_function, pack_tiles

# tuning arguments the reference passes to its GEMV (modules/linear.py:176-185); validated, then unused
_GEMV_KWARGS = {
    "num_thread_stage1": 128, "num_thread_stage2": 128,
    "num_row_per_warp_stage1": 2, "num_row_per_warp_stage2": 2,
    "num_acc_stage1": 1, "num_acc_stage2": 1,
    "num_pipeline_stage1": 8, "num_pipeline_stage2": 8,
}


class NanoQuantLinear(nn.Module):
    """y = scale_post * (U @ (scale_mid * (V @ (scale_pre * x)))) with ±1 ``V [R, N]``, ``U [M, R]``."""

    def __init__(self, in_features: int, out_features: int, rank: int, has_scale_mid: bool = True,
                 bias: bool = False, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_parameter("weight", None)
        self.bias = nn.Parameter(torch.zeros(out_features, device=device)) if bias else None
        self.init_for_inference(rank, has_scale_mid)

    # reference: modules/linear.py:86-99 (allocates the parameters that load_state_dict fills)
    def init_for_inference(self, rank, has_scale_mid=False):
        self.rank = rank
        self.do_train = False
        self._binarized = True
        self.dtype = torch.bfloat16
        if "weight" in self._parameters:
            del self._parameters["weight"]
        self.register_parameter("weight", None)
        bias = getattr(self, "bias", None)
        device = bias.device if bias is not None else torch.device("cpu")
        shapes = {"scale_pre": (1, self.in_features), "scale_post": (1, self.out_features),
                  "V": (self.rank, self.in_features), "U": (self.out_features, self.rank)}
        if has_scale_mid:
            shapes["scale_mid"] = (1, self.rank)
        elif hasattr(self, "scale_mid"):
            delattr(self, "scale_mid")
        for name, shape in shapes.items():
            setattr(self, name, nn.Parameter(torch.empty(shape, device=device, dtype=self.dtype),
                                             requires_grad=False))

    # ------------------------------------------------------------------ forward
    def forward(self, x):
        if not getattr(self, "do_kernel_inference", False):
            raise RuntimeError("NanoQuantLinear: call _prepare_kernel() first; this package implements the "
                               "CUDA kernel inference path only (no dense PyTorch forward)")
        orig_dtype = x.dtype
        if x.dtype != self.dtype:
            x = x.to(self.dtype)
        original_shape = None
        if x.ndim == 3:
            original_shape = x.shape
            x = x.contiguous().view(-1, x.size(-1))
        elif x.ndim == 2:
            x = x.contiguous()
        else:
            raise ValueError(f"Expected 2D or 3D input tensor, got {x.ndim}D")
        bias = getattr(self, "bias", None)
        if bias is not None:
            # The reference adds the bias only on its PyTorch path (modules/linear.py:148-149) and drops it on the
            # kernel branches (:121-141).  Here it rides in the kernel's epilogue (fp32, behind the output scale).
            from .. import ops
            if bias.dtype != self.dtype:
                bias = bias.to(self.dtype)
            if self.kernel_type == "gemv":
                y = ops.linear_forward(x, self.scale_pre, self.V_int8, self.scale_mid, self.U_int8, self.scale_post,
                                       self.rank, bias=bias)
            else:
                y = ops.linear_forward(x, self.s1, self.V_int8, self.s2, self.U_int8, self.s3, self.rank, bias=bias)
        elif self.kernel_type == "gemv":
            y = self.kernel_forward(x, self.scale_pre, self.V_int8, self.scale_mid, self.U_int8,
                                    self.scale_post, **self.kernel_kwargs)
        elif self.kernel_type == "gemm":
            y = self.kernel_forward(x, self.V_int8, self.U_int8, self.s1, self.s2, self.s3, self.workspace)
        else:
            raise ValueError(f"Unknown kernel_type: {self.kernel_type}")
        if original_shape is not None:
            y = y.view(original_shape[0], original_shape[1], -1)
        return y.to(orig_dtype) if y.dtype != orig_dtype else y

    # ------------------------------------------------------------ kernel set-up
    def _squeeze_scales(self, dtype):
        self.scale_pre = nn.Parameter(self.scale_pre.to(dtype).reshape(-1), requires_grad=False)
        self.scale_post = nn.Parameter(self.scale_post.to(dtype).reshape(-1), requires_grad=False)
        mid = getattr(self, "scale_mid", None)
        self.scale_mid = None if mid is None else nn.Parameter(mid.to(dtype).reshape(-1), requires_grad=False)

    def _prepare_kernel(self, kernel_type="gemv", dtype=torch.float16):
        """One-time repack for kernel inference (reference ``modules/linear.py:152-204``).
        ``gemv``: ``V_int8`` / ``U_int8`` become the kernel's tile layout."""
        if kernel_type not in ("gemv", "gemm"):
            raise ValueError("kernel_type must be one of ['gemv', 'gemm'].")
        self.do_kernel_inference = True
        self.kernel_type = kernel_type
        self.dtype = dtype
        self._squeeze_scales(dtype)
        if hasattr(self, "V"):     # dense +-1 factors -> the kernels' tile layout (one copy of the weights, both kernels)
            dev = self.V.device
            v_bits = binary_packer(self.V.to(torch.int8), method="half2")
            u_bits = binary_packer(self.U.to(torch.int8), method="half2")
            self.V_int8 = pack_tiles(v_bits, (self.rank, self.in_features), "half2").to(dev)
            self.U_int8 = pack_tiles(u_bits, (self.out_features, self.rank), "half2").to(dev)
            delattr(self, "U")
            delattr(self, "V")
        # the tiles pad the rank to 16: the operators read the exact rank from here when there is no scale_mid
        self.V_int8._nq_rows, self.V_int8._nq_cols = self.rank, self.in_features
        self.U_int8._nq_rows, self.U_int8._nq_cols = self.out_features, self.rank
        if kernel_type == "gemv":
            self.kernel_forward = get_kernel_function("nanoquant", dtype, kernel_type="dynamic")
            self.kernel_kwargs = dict(_GEMV_KWARGS)
        else:
            # Same attribute names and call protocol as the reference (modules/linear.py:186-202: V_int8, U_int8,
            # s1..s3, workspace -> marlin_nanoquant_forward).  The reference keeps Marlin-fragment words and
            # permuted scales there; this module keeps the tile layout and plain scales, which the operator takes
            # as they are (operands made by the reference's own packer are converted by the operator instead).
            if self.scale_mid is None:
                self.scale_mid = nn.Parameter(torch.ones(self.rank, device=self.scale_pre.device, dtype=dtype),
                                              requires_grad=False)
            self.s1, self.s2, self.s3 = self.scale_pre, self.scale_mid, self.scale_post
            self.workspace = torch.zeros(max(self.rank, self.out_features) // 128 * 32 + 32, dtype=torch.int32,
                                         device=self.V_int8.device)
            for key in ("scale_pre", "scale_mid", "scale_post"):
                delattr(self, key)
            import binary_kernels  # noqa: F401
            self.kernel_forward = torch.ops.binary_kernels.marlin_nanoquant_forward
        # the kernels' scratch of this device is sized for its largest layer before the first forward
        from .. import ops, _lib
        ops.reserve_scratch(self.V_int8.device, _lib.lib().nq_linear_scratch_bytes(
            64, self.in_features, self.rank, self.out_features))

    def fold_input_scale(self, weight: torch.Tensor) -> None:
        """Multiply ``scale_pre`` by a per-input-column weight (fp32 product, stored in the scale's dtype).

        For the RMSNorm that feeds this linear in a decoder layer: ``linear(norm(x) * w)`` becomes
        ``linear'(norm(x))`` with ``scale_pre' = scale_pre * w``, which removes an elementwise pass and one
        rounding of the activations.  Valid before and after ``_prepare_kernel`` (for ``kernel_type="gemm"`` the
        input scale then lives in ``s1``, in plain order)."""
        target = self.scale_pre if hasattr(self, "scale_pre") else self.s1
        w = weight.detach().reshape(-1).to(device=target.device, dtype=torch.float32)
        if w.numel() != self.in_features:
            raise ValueError(f"fold_input_scale: expected {self.in_features} weights, got {w.numel()}")
        with torch.no_grad():
            folded = target.detach().float() * w.view_as(target)
            target.copy_(folded.to(target.dtype))

    def load_packed(self, V_packed, V_shape, U_packed, U_shape, scale_pre, scale_post, scale_mid=None,
                    dtype=torch.bfloat16, device="cuda", kernel_type="gemv"):
        """Checkpoint tensors (``lsb_first`` words, reference ``modules/linear.py:288-303``)
        straight to the kernel's tile layout: no dense ±1 matrices are created,
        unlike ``src/nanoquant/utils/load_utils.py:279-287``."""
        R, N = (int(v) for v in V_shape)
        M, R2 = (int(v) for v in U_shape)
        if (N, M) != (self.in_features, self.out_features) or R != R2:
            raise ValueError(f"packed shapes V{(R, N)} U{(M, R2)} do not match this layer")
        self.rank = R
        for name in ("V", "U"):
            if hasattr(self, name):
                delattr(self, name)
        self.V_int8 = pack_tiles(V_packed.to(device), (R, N), "lsb_first")
        self.U_int8 = pack_tiles(U_packed.to(device), (M, R), "lsb_first")
        self.scale_pre = nn.Parameter(scale_pre.to(device), requires_grad=False)
        self.scale_post = nn.Parameter(scale_post.to(device), requires_grad=False)
        if scale_mid is not None:
            self.scale_mid = nn.Parameter(scale_mid.to(device), requires_grad=False)
        elif hasattr(self, "scale_mid"):
            delattr(self, "scale_mid")
        self._prepare_kernel(kernel_type, dtype)

    # --------------------------------------------------------- checkpoint format
    def pack_weights(self):
        """``{V,U}_packed`` (``lsb_first`` int32 words) and ``{V,U}_shape`` (int64),
        the reference checkpoint keys (``modules/linear.py:288-303``)."""
        out = {}
        for name in ("V", "U"):
            p = getattr(self, name, None)
            if p is None:
                continue
            sign = torch.where(p.data < 0, -1, 1).to(torch.int8)
            out[f"{name}_packed"] = binary_packer(sign)
            out[f"{name}_shape"] = torch.tensor(p.shape, dtype=torch.long)
        return out

    def state_dict(self, *args, **kwargs):
        state = super().state_dict(*args, **kwargs)
        prefix = kwargs.get("prefix", "")
        for k in [k for k in state if ".V" in k or ".U" in k or k in (prefix + "V", prefix + "U")]:
            del state[k]
        for k, v in self.pack_weights().items():
            state[prefix + k] = v
        return state
