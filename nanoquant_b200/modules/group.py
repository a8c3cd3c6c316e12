"""Launch groups: the linears of a decoder layer that share their input (q/k/v, gate/up) in ONE kernel launch.

The reference runs one operator call per projection (``modules/linear.py:121-132``, two kernel launches each);
at decode batch sizes a launch is a chain of latencies, so the step time is set by the number of launches.
``LinearGroup`` issues ``nq_gemv_group_fwd`` (up to four tokens) or ``nq_gemm_group_fwd`` for up to four
prepared :class:`~nanoquant_b200.modules.linear.NanoQuantLinear` modules, with their biases and optional
residuals in the kernel's epilogue.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .linear import NanoQuantLinear


class LinearGroup:
    """Up to four prepared quantised linears evaluated by one launch per call."""

    def __init__(self, modules: Sequence[NanoQuantLinear]):
        if not 1 <= len(modules) <= 4:
            raise ValueError("a launch group holds one to four linears")
        for m in modules:
            if not getattr(m, "do_kernel_inference", False):
                raise RuntimeError("LinearGroup: call _prepare_kernel() on every module first")
        self.modules = list(modules)
        self.dtype = modules[0].dtype
        if any(m.dtype != self.dtype for m in modules):
            raise ValueError("the linears of a group share one dtype")
        # scratch for this group at decode batches and at up to 64 tokens, reserved now: a forward (or a stream
        # capture) then only reads the buffer's address
        shapes = [(m.in_features, m.rank, m.out_features) for m in self.modules]
        device = self.modules[0].scale_post.device
        ops.reserve_scratch(device, max(ops.group_scratch_bytes(shapes, T) for T in (4, 24, 64)))

    @staticmethod
    def _layer(m: NanoQuantLinear):
        if m.kernel_type == "gemv":
            return (m.scale_pre, m.V_int8, m.scale_mid, m.U_int8, m.scale_post, m.rank)
        return (m.s1, m.V_int8, m.s2, m.U_int8, m.s3, m.rank)

    def __call__(self, x, residuals: Optional[Sequence[Optional[torch.Tensor]]] = None,
                 out: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
        """`x`: one ``[..., N]`` tensor for all linears, or one per linear.  Returns one ``[..., M_i]`` tensor per
        linear (column views of one buffer)."""
        xs = list(x) if isinstance(x, (list, tuple)) else [x] * len(self.modules)
        lead = xs[0].shape[:-1]
        xs2 = []
        for xi in xs:
            if xi.dtype != self.dtype:
                xi = xi.to(self.dtype)
            xi = xi.reshape(-1, xi.size(-1))
            xs2.append(xi if xi.stride(-1) == 1 else xi.contiguous())
        T = xs2[0].size(0)
        res2 = None
        if residuals is not None:
            res2 = [None if r is None else r.reshape(-1, r.size(-1)) for r in residuals]
        biases = []
        for m in self.modules:
            b = getattr(m, "bias", None)
            biases.append(None if b is None else (b if b.dtype == self.dtype else b.to(self.dtype)))
        views = ops.group_forward(xs2, [self._layer(m) for m in self.modules], T, self.dtype, xs2[0].device,
                                  biases, res2, out)
        return [v.reshape(*lead, v.size(-1)) if len(lead) != 1 else v for v in views]
