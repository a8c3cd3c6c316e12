"""Helpers shared by the GPU parity tests: seeded layers, oracle evaluation."""
import numpy as np
import torch

from oracle import nanoquant_oracle as oc

# Parity bar: max|y - y64| / max|y64| <= 2e-3 against the fp64 oracle.  A bf16
# output cannot represent the result better than half a unit in the last place of
# its 8-bit significand (2^-8 of the element), so for bf16 that representation
# error is allowed on top; fp16 (2^-11) fits inside the bar.
TOL = {torch.float16: 2e-3, torch.bfloat16: 2e-3 + 2.0 ** -8}


def np_to_torch(a, dtype, device="cuda"):
    """numpy fp16/fp32 array -> torch tensor of `dtype` with the same values when representable."""
    return torch.from_numpy(np.ascontiguousarray(a).astype(np.float32)).to(dtype).to(device)


def exact_np(t):
    """torch fp16/bf16 tensor -> float64 numpy with the exact stored values."""
    return t.detach().float().cpu().numpy().astype(np.float64)


def make_layer(N, R, M, T, dtype, seed=0, has_mid=True, device="cuda"):
    d = oc.synth_linear(N, R, M, T, seed=seed)
    L = {
        "V": d["V"], "U": d["U"],
        "x": np_to_torch(d["x"], dtype, device),
        "s_pre": np_to_torch(d["s_pre"], dtype, device),
        "s_mid": np_to_torch(d["s_mid"], dtype, device) if has_mid else None,
        "s_post": np_to_torch(d["s_post"], dtype, device),
        "N": N, "R": R, "M": M, "T": T,
    }
    L["y64"] = oc.forward_fp64(exact_np(L["x"]), L["V"], L["U"], exact_np(L["s_pre"]),
                               exact_np(L["s_mid"]) if has_mid else None, exact_np(L["s_post"]))
    return L


def half2_bits(w, device="cuda"):  # noqa: D401
    return torch.from_numpy(oc.pack_rows(w, "half2")).to(device)
