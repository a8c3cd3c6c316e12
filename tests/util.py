"""Helpers shared by the GPU parity tests: seeded layers, oracle evaluation."""
import numpy as np
import torch

from oracle import nanoquant_oracle as oc

# Parity bar against the fp64 oracle, element by element:
#     |y - y64| <= 2e-3 * max|y64| + half a unit in the last place of the output type at that element
# (`parity_excess` / `assert_parity` below).  The representation error of a rounded output belongs to the
# element (2^-9 of it for bf16, 2^-12 for fp16), not to the largest one, so a 2e-3 error before the final rounding
# cannot hide behind it.  TOL is the older max-normalised bar, kept for comparisons between two rounded results.
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


def tiles_on_gpu(w, device="cuda"):
    """Dense ±1 int8 matrix (numpy) -> the kernels' tile layout, packed on the GPU (the packers are pinned
    bit for bit elsewhere); for layers too large to pack in numpy within a test's time."""
    from nanoquant_b200.kernel import utils as ku
    bits = ku.pack_binary_gemv(torch.from_numpy(np.ascontiguousarray(w)).to(device), method="half2")
    return ku.pack_tiles(bits, w.shape, "half2")


def make_group(shapes, T, dtype, seed=0, no_mid=(), device="cuda"):
    """Linears of one launch group: every linear with the same N shares one activation tensor (as q/k/v or
    gate/up of a decoder layer do); `no_mid` lists the indices that have no middle scale."""
    layers, x_by_n = [], {}
    for i, (N, R, M) in enumerate(shapes):
        L = make_layer(N, R, M, T, dtype, seed=seed + 17 * i, has_mid=i not in no_mid, device=device)
        if N in x_by_n:
            L["x"] = x_by_n[N]
            L["y64"] = oc.forward_fp64(exact_np(L["x"]), L["V"], L["U"], exact_np(L["s_pre"]),
                                       exact_np(L["s_mid"]) if L["s_mid"] is not None else None, exact_np(L["s_post"]))
        else:
            x_by_n[N] = L["x"]
        layers.append(L)
    return layers


def elementwise_bound(y64, dtype, rel=2e-3, y=None):
    """Per-element parity bound: `rel` of the largest reference magnitude plus half a unit in the last
    place of the output type at that element (the representation error belongs to the element; the
    binade is that of the larger of reference and result, which differ when they straddle a power of two)."""
    y64 = np.asarray(y64, np.float64)
    bits = 11 if dtype == torch.float16 else 8
    mag = np.maximum(np.abs(y64), 2.0 ** -126)
    if y is not None:
        mag = np.maximum(mag, np.abs(np.asarray(y, np.float64)))
    half_ulp = 2.0 ** (np.floor(np.log2(mag)) - bits)
    return rel * np.max(np.abs(y64)) + half_ulp


def parity_excess(y, y64, dtype, rel=2e-3):
    """max over the elements of |y - y64| minus the element's bound; parity holds when this is <= 0."""
    y = np.asarray(y, np.float64)
    return float((np.abs(y - np.asarray(y64, np.float64)) - elementwise_bound(y64, dtype, rel, y)).max())


def assert_parity(y, y64, dtype, rel=2e-3, what=""):
    """|y - y64| <= rel * max|y64| + half an ulp of `dtype` at y64, element by element."""
    y = np.asarray(y, np.float64)
    excess = np.abs(y - np.asarray(y64, np.float64)) - elementwise_bound(y64, dtype, rel, y)
    worst = float(excess.max())
    assert worst <= 0, (f"{what}: element exceeds {rel:g}*max|y64| + half ulp by {worst:.3e} "
                        f"(max-normalised error {oc.rel_err(y, y64):.3e})")
