"""Compressed checkpoints of a model: save and load, the inference side of the reference's
``src/nanoquant/utils/load_utils.py``.

Same checkpoint format (``get_compressed_state_dict``, reference ``load_utils.py:216-241``: per quantised
linear ``<name>.V_packed`` / ``<name>.V_shape`` / ``<name>.U_packed`` / ``<name>.U_shape`` with ``lsb_first``
words, ``scale_pre`` / ``scale_post`` / optional ``scale_mid`` / optional ``bias``; every other parameter under
its own name).  Loading differs on purpose: the reference unpacks every factor to a dense matrix on the
CPU (``load_utils.py:279-287``, 16 bytes of host memory traffic per weight) and re-packs it on the GPU in
``_prepare_kernel``; here the packed words go to the GPU as they are and one kernel (``nq_rows_to_tiles``)
turns them into the runtime layout: no dense +-1 matrix exists at any point.
"""
from __future__ import annotations

import inspect
import os
from collections import OrderedDict
from typing import Dict, Optional

import torch
import torch.nn as nn

from ..modules.linear import NanoQuantLinear

_LINEAR_KEYS = ("V_packed", "V_shape", "U_packed", "U_shape", "scale_pre", "scale_post", "scale_mid", "bias")


def get_compressed_state_dict(model: nn.Module) -> "OrderedDict[str, torch.Tensor]":
    """State dict of `model` with every ``NanoQuantLinear`` in its packed form (reference
    ``load_utils.py:216-241``); modules already prepared for kernel inference have no dense factors left and
    cannot be saved."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    quantised = {name for name, mod in model.named_modules() if isinstance(mod, NanoQuantLinear)}
    for name, param in model.named_parameters():
        if name.rsplit(".", 1)[0] not in quantised:
            out[name] = param.data
    for name, mod in model.named_modules():
        if isinstance(mod, NanoQuantLinear):
            if not hasattr(mod, "V"):
                raise RuntimeError(f"{name}: prepared for kernel inference, the dense factors are gone")
            out.update(mod.state_dict(prefix=name + "."))
    return out


def load_compressed_state_dict(model: nn.Module, sd: Dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16,
                               device="cuda", kernel_type: str = "gemv", skip=("lm_head",)) -> nn.Module:
    """Fill `model` from a compressed state dict and prepare it for kernel inference.

    Every ``nn.Linear`` whose name has ``<name>.V_packed`` in `sd` (and is not in `skip`, as the reference keeps
    ``lm_head`` dense, ``load_utils.py:322``) becomes a :class:`NanoQuantLinear` (class swap as in
    ``load_utils.py:319-327``) and takes its packed words straight into the kernels' tile layout on `device`;
    everything else goes through ``load_state_dict(strict=False)``.  Returns `model` (moved to `device`)."""
    rest = {k: v for k, v in sd.items() if k.rsplit(".", 1)[-1] not in _LINEAR_KEYS or
            (k.rsplit(".", 1)[0] + ".V_packed") not in sd}
    for name, module in list(model.named_modules()):
        base = name + "."
        if base + "V_packed" not in sd or any(s in name for s in skip):
            continue
        if type(module) is nn.Linear:
            module.__class__ = NanoQuantLinear
        elif not isinstance(module, NanoQuantLinear):
            raise TypeError(f"{name}: packed factors in the checkpoint, but the module is a {type(module).__name__}")
        rank = int(sd[base + "V_shape"][0])
        mid = sd.get(base + "scale_mid")
        module.init_for_inference(rank=rank, has_scale_mid=mid is not None)
        bias = sd.get(base + "bias")
        if bias is not None:
            module.bias = nn.Parameter(bias.to(device=device, dtype=dtype), requires_grad=False)
        elif getattr(module, "bias", None) is not None:
            module.bias = None
        sq = lambda t: t.reshape(-1)
        module.load_packed(sd[base + "V_packed"], sd[base + "V_shape"], sd[base + "U_packed"], sd[base + "U_shape"],
                           sq(sd[base + "scale_pre"]), sq(sd[base + "scale_post"]), sq(mid) if mid is not None else None,
                           dtype=dtype, device=device, kernel_type=kernel_type)
    missing, unexpected = model.load_state_dict(rest, strict=False)
    unexpected = [k for k in unexpected]
    if unexpected:
        raise KeyError(f"checkpoint entries without a home in the model: {unexpected[:8]}")
    # move what is not a prepared quantised linear (their tensors are on `device` already)
    for mod in model.modules():
        if isinstance(mod, NanoQuantLinear):
            continue
        for pname, p in list(mod.named_parameters(recurse=False)):
            if p is not None and p.device.type != torch.device(device).type:
                setattr(mod, pname, nn.Parameter(p.data.to(device), requires_grad=False))
        for bname, b in list(mod.named_buffers(recurse=False)):
            if b is not None and b.device.type != torch.device(device).type:
                setattr(mod, bname, b.to(device))
    return model


def load_compressed_checkpoint(model: nn.Module, checkpoint_path: str, dtype: torch.dtype = torch.bfloat16,
                               device="cuda", kernel_type: str = "gemv") -> nn.Module:
    """``torch.load`` (memory-mapped, weights only where the installed torch allows: reference
    ``load_utils.py:244-262``) followed by :func:`load_compressed_state_dict`."""
    if not os.path.exists(checkpoint_path):
        raise FileNotFoundError(f"Could not find model weights at {checkpoint_path}")
    kwargs = {"map_location": "cpu"}
    sig = inspect.signature(torch.load)
    if "mmap" in sig.parameters:
        kwargs["mmap"] = True
    if "weights_only" in sig.parameters:
        kwargs["weights_only"] = True
    sd = torch.load(checkpoint_path, **kwargs)
    if not isinstance(sd, dict):
        raise TypeError(f"Expected a state_dict dict from {checkpoint_path}, got {type(sd)}")
    return load_compressed_state_dict(model, sd, dtype=dtype, device=device, kernel_type=kernel_type)
