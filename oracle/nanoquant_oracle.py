"""CPU oracle for the NanoQuant binary low-rank quantised linear.

TEST INFRASTRUCTURE ONLY.  This file restates, in numpy, the arithmetic of the
reference implementation (SamsungLabs/NanoQuant) for the inference hot path so
that the CUDA kernels of ``nanoquant_b200`` can be checked against it.  It is
imported only by the tests, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The product path
never imports it and never falls back to it.

Parity pin: every function below is compared, in ``tests/test_oracle_golden.py``,
with fixtures under ``tests/golden/`` that were produced by importing and running
the reference's own Python code (``tests/golden/make_golden.py``).

Conventions (reference ``src/nanoquant/kernel/utils.py:87-96``): a weight of
+1 is stored as bit 0, a weight of -1 as bit 1, padding columns are +1.

Shapes use N = in_features, R = rank, M = out_features, T = tokens.  The module
holds ``V [R, N]`` (applied first) and ``U [M, R]`` (applied second).
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------
# bit position tables
# ----------------------------------------------------------------------------

def _bitpos_lsb() -> np.ndarray:
    """Element k of a 32-column group lands in bit k
    (reference ``kernel/utils.py:99-100``)."""
    return np.arange(32, dtype=np.uint32)


def _bitpos_half2() -> np.ndarray:
    """Element 2j lands in bit 15-j, element 2j+1 in bit 31-j, j = 0..15
    (reference ``kernel/utils.py:101-104``).  After a left shift by j the two
    bits sit on the sign positions of an fp16/bf16 pair."""
    e = np.arange(32, dtype=np.uint32)
    return (15 - (e >> 1) + 16 * (e & 1)).astype(np.uint32)


_BITPOS = {"lsb_first": _bitpos_lsb, "half2": _bitpos_half2}


def _positions(method: str) -> np.ndarray:
    if method not in _BITPOS:
        raise ValueError(
            f"Unsupported method: '{method}'. Supported methods are 'lsb_first', 'half2'.")
    return _BITPOS[method]()


# ----------------------------------------------------------------------------
# row packers (checkpoint layout ``lsb_first`` and GEMV layout ``half2``)
# ----------------------------------------------------------------------------

def pack_rows(w: np.ndarray, method: str = "lsb_first") -> np.ndarray:
    """±1 int8 ``[rows, cols]`` -> int32 ``[rows, ceil(cols/32)]``.

    Follows reference ``pack_binary_gemv`` (``kernel/utils.py:51-113``).
    """
    if w.dtype != np.int8:
        raise TypeError("Input tensor must be int8.")
    pos = _positions(method)
    rows, cols = w.shape
    words = (cols + 31) // 32
    neg = np.zeros((rows, words * 32), dtype=np.uint32)
    neg[:, :cols] = (w < 0)
    neg = neg.reshape(rows, words, 32)
    out = np.zeros((rows, words), dtype=np.uint32)
    for e in range(32):
        out |= neg[:, :, e] << pos[e]
    return out.view(np.int32)


def unpack_rows(packed: np.ndarray, shape, method: str = "lsb_first") -> np.ndarray:
    """Inverse of :func:`pack_rows` (reference ``unpack_binary_gemv``,
    ``kernel/utils.py:116-183``)."""
    if packed.ndim != 2:
        raise ValueError(
            f"Unsupported packed tensor format. Expected 2D tensor, got {packed.ndim} dimensions.")
    rows, cols = int(shape[0]), int(shape[1])
    words = (cols + 31) // 32
    if packed.shape != (rows, words):
        raise ValueError(
            f"Unsupported packed tensor shape. Expected ({rows}, {words}), got {packed.shape}.")
    pos = _positions(method)
    u = packed.view(np.uint32) if packed.dtype == np.int32 else packed.astype(np.uint32)
    bits = (u[:, :, None] >> pos[None, None, :]) & 1
    bits = bits.reshape(rows, words * 32)[:, :cols]
    return (1 - 2 * bits.astype(np.int8)).astype(np.int8)


# ----------------------------------------------------------------------------
# Marlin-fragment packer (API parity with the reference GEMM path)
# ----------------------------------------------------------------------------

def pack_marlin_bits(w: np.ndarray) -> np.ndarray:
    """±1 ``[out, in]`` (out % 64 == 0, in % 16 == 0) -> int32 ``[in/16, out/2]``.

    With out = 64*to + 16*o16 + 8*o8 + o1 and in = 16*tr + 8*r8 + 2*r2 + r1 the
    weight lands at row ``tr``, column ``32*to + 4*o1 + r2`` and bit
    ``15 - 4*o16 - 2*o8 - r8 + 16*r1`` (reference ``pack_binary_marlin``,
    ``kernel/utils.py:191-205``).
    """
    out_f, in_f = w.shape
    if out_f % 64 or in_f % 16:
        raise ValueError("marlin packing needs out % 64 == 0 and in % 16 == 0")
    o = np.arange(out_f)[:, None]
    i = np.arange(in_f)[None, :]
    to, o16, o8, o1 = o // 64, (o // 16) % 4, (o // 8) % 2, o % 8
    tr, r8, r2, r1 = i // 16, (i // 8) % 2, (i // 2) % 4, i % 2
    row = np.broadcast_to(tr, w.shape)
    col = 32 * to + 4 * o1 + r2
    bit = (15 - 4 * o16 - 2 * o8 - r8 + 16 * r1).astype(np.uint32)
    B = np.zeros((in_f // 16, out_f // 2), dtype=np.uint32)
    np.bitwise_or.at(B, (row, col), (w < 0).astype(np.uint32) << bit)
    return B.view(np.int32)


def marlin_perm_scale_in(s: np.ndarray) -> np.ndarray:
    """Per group of 16: new[4b + 2a + c] = old[8a + 2b + c]
    (reference ``kernel/utils.py:206-207``)."""
    return np.ascontiguousarray(s.reshape(-1, 2, 4, 2).transpose(0, 2, 1, 3)).reshape(-1)


def marlin_perm_scale_out(s: np.ndarray) -> np.ndarray:
    """Per group of 32: new[8b + 2a + c] = old[8a + 2b + c]
    (reference ``kernel/utils.py:208-209``)."""
    return np.ascontiguousarray(s.reshape(-1, 4, 4, 2).transpose(0, 2, 1, 3)).reshape(-1)


MARLIN_MIN_MAX_PAR = 32


def pack_marlin(w: np.ndarray, scale_in: np.ndarray, scale_out: np.ndarray):
    """Reference ``pack_binary_marlin`` (``kernel/utils.py:186-214``)."""
    B = pack_marlin_bits(w)
    s_in = marlin_perm_scale_in(scale_in)
    s_out = marlin_perm_scale_out(scale_out)
    return B, s_in, s_out, s_out.size // 128 * MARLIN_MIN_MAX_PAR


def pack_marlin_fused(V_sign: np.ndarray, U_sign: np.ndarray, scale_g, scale_l, scale_h):
    """Reference ``pack_binary_marlin_fused`` (``kernel/utils.py:217-284``).

    ``V_sign`` is ``[N, R]``, ``U_sign`` is ``[R, M]``.  The rank is padded to a
    multiple of 256 with +1 signs and zero ``scale_l``.
    """
    N = scale_g.shape[0]
    R = scale_l.shape[0] if scale_l is not None else U_sign.shape[0]
    M = scale_h.shape[0]
    N, R, M = [(d + 31) // 32 * 32 for d in (N, R, M)]
    R_pad = (R + 255) // 256 * 256
    if R_pad > R:
        pad = R_pad - R
        V_sign = np.concatenate([V_sign, np.ones((N, pad), np.int8)], axis=1)
        U_sign = np.concatenate([U_sign, np.ones((pad, M), np.int8)], axis=0)
        if scale_l is not None:
            scale_l = np.concatenate([scale_l, np.zeros(pad, scale_l.dtype)])
    V_bits, s_g, s_l, ws_v = pack_marlin(np.ascontiguousarray(V_sign.T), scale_g, scale_l)
    U_bits, _, s_h, ws_u = pack_marlin(np.ascontiguousarray(U_sign.T), scale_l, scale_h)
    workspace = np.zeros(max(ws_v, ws_u), dtype=np.int32)
    return V_bits, U_bits, s_g, s_l, s_h, workspace


# ----------------------------------------------------------------------------
# forward
# ----------------------------------------------------------------------------

def forward_fp64(x, V, U, s_pre, s_mid, s_post, bias=None) -> np.ndarray:
    """The reference's dequantise-then-matmul forward evaluated in float64.

    ``y = (((x * s_pre) @ V.T) * s_mid) @ U.T * s_post`` (+ bias), reference
    ``NanoQuantLinear._compute_forward`` (``modules/linear.py:248-257``) and the
    bias add at ``modules/linear.py:148-149``.  Inputs are taken at the exact
    values they have in their storage dtype.
    """
    x = np.asarray(x, dtype=np.float64)
    t = (x * np.asarray(s_pre, np.float64)) @ np.asarray(V, np.float64).T
    if s_mid is not None:
        t = t * np.asarray(s_mid, np.float64)
    y = t @ np.asarray(U, np.float64).T
    y = y * np.asarray(s_post, np.float64)
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y


def dense_forward_fp64(x, W, bias=None) -> np.ndarray:
    """``F.linear(x, W, bias)`` in float64 on the exact stored values: the un-quantised ``lm_head`` the
    reference's decode loop calls once per token (``utils/load_utils.py:322`` keeps it an ``nn.Linear``)."""
    y = np.asarray(x, np.float64) @ np.asarray(W, np.float64).T
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    return y


def forward_from_packed(x, Vp, Up, s_pre, s_mid, s_post, N, R, M, method="half2"):
    """:func:`forward_fp64` on packed factors ``Vp [R, N/32]``, ``Up [M, R/32]``."""
    V = unpack_rows(np.asarray(Vp), (R, N), method)
    U = unpack_rows(np.asarray(Up), (M, R), method)
    return forward_fp64(x, V, U, s_pre, s_mid, s_post)


def rel_err(y, y64) -> float:
    """Parity metric: ``max|y - y64| / max|y64|``."""
    y64 = np.asarray(y64, np.float64)
    d = np.max(np.abs(np.asarray(y, np.float64) - y64))
    return float(d / max(np.max(np.abs(y64)), 1e-300))


# ----------------------------------------------------------------------------
# rank-from-bits formula and the synthetic workloads
# ----------------------------------------------------------------------------

def rank_for_bits(in_f: int, out_f: int, bits: float, num_scales: int = 2) -> int:
    """Reference ``calculate_ranks`` (``utils/utils.py:128-182``)."""
    budget = in_f * out_f * bits
    s = in_f + out_f
    r = (budget - 16 * s) / (s + 16) if num_scales == 3 else budget / s - 16
    r = (int(r) // 32) * 32
    r = max(r if r else 32, 32)
    return min(r, in_f, out_f)


def synth_linear(N, R, M, T, seed=0, dtype=np.float16):
    """Seeded synthetic layer in the value distributions the workloads specify:
    i.i.d. ±1 signs (p = 0.5), scales ``(U[0,1) + 0.5) * 0.01`` rounded to
    ``dtype``, activations N(0, 1) rounded to ``dtype``."""
    g = np.random.default_rng(seed)
    V = (g.integers(0, 2, size=(R, N), dtype=np.int8) * 2 - 1).astype(np.int8)
    U = (g.integers(0, 2, size=(M, R), dtype=np.int8) * 2 - 1).astype(np.int8)
    s_pre = ((g.random(N) + 0.5) * 0.01).astype(dtype)
    s_mid = ((g.random(R) + 0.5) * 0.01).astype(dtype)
    s_post = ((g.random(M) + 0.5) * 0.01).astype(dtype)
    x = g.standard_normal((T, N)).astype(dtype)
    return dict(V=V, U=U, s_pre=s_pre, s_mid=s_mid, s_post=s_post, x=x)


# ----------------------------------------------------------------------------
# timed CPU baseline (the reference's PyTorch path restated with torch on CPU)
# ----------------------------------------------------------------------------

def torch_cpu_forward(x, V, U, s_pre, s_mid, s_post):
    """Dense ±1 matmul forward with torch CPU tensors in their own dtype, the
    four lines of reference ``modules/linear.py:252-256``.  Used only as the
    timed CPU baseline; ``V``/``U`` are dense ±1 tensors in the compute dtype as
    the reference module keeps them (``modules/linear.py:69-76``)."""
    import torch.nn.functional as F
    t = F.linear(x * s_pre, V)
    if s_mid is not None:
        t = t * s_mid
    y = F.linear(t, U)
    return y * s_post
