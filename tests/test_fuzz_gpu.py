"""Seeded random shapes through the dispatcher (GEMV up to four tokens, split-K GEMM, GEMM) against the fp64
oracle: ragged input widths, ranks, output widths and token counts, both dtypes."""
import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc
from tests.util import parity_excess, TOL, exact_np, half2_bits, make_layer

pytestmark = pytest.mark.gpu


def _cases(seed, n):
    g = np.random.default_rng(seed)
    out = []
    for i in range(n):
        T = int(g.choice([1, 2, 3, 4, 5, 7, 8, 13, 16, 33, 64, 65, 100, 129, 200]))
        if i % 5 == 0:   # anything goes: unaligned widths take the scalar paths of the GEMV
            N, R, M = int(g.integers(1, 700)), int(g.integers(1, 300)), int(g.integers(1, 700))
            T = min(T, 8)
        else:
            N, R, M = 8 * int(g.integers(1, 260)), 8 * int(g.integers(1, 130)), int(g.integers(1, 2100))
        out.append((N, R, M, T, torch.float16 if i % 2 else torch.bfloat16))
    return out


@pytest.mark.parametrize("case", _cases(2024, 40), ids=lambda c: f"{c[0]}x{c[1]}x{c[2]}-T{c[3]}-{str(c[4])[6:]}")
def test_random_shapes_vs_oracle(case):
    from nanoquant_b200 import ops
    from nanoquant_b200.kernel import utils as ku
    N, R, M, T, dtype = case
    L = make_layer(N, R, M, T, dtype, seed=N * 7 + R * 3 + M + T)
    vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
    y = ops.linear_forward(L["x"], L["s_pre"], vt, L["s_mid"], ut, L["s_post"], R)
    y2 = ops.linear_forward(L["x"], L["s_pre"], vt, L["s_mid"], ut, L["s_post"], R)
    assert y.shape == (T, M) and torch.equal(y, y2)
    assert parity_excess(exact_np(y), L["y64"], dtype) <= 0


def _epilogue_cases(seed, n):
    g = np.random.default_rng(seed)
    out = []
    for i in range(n):
        T = int(g.choice([1, 4, 6, 20, 25, 48, 130, 300, 600]))
        N, R, M = 8 * int(g.integers(4, 200)), 8 * int(g.integers(2, 120)), int(g.integers(1, 1500))
        out.append((N, R, M, T, torch.bfloat16 if i % 3 else torch.float16, bool(i % 2), i % 4 == 0))
    return out


@pytest.mark.parametrize("case", _epilogue_cases(77, 24),
                         ids=lambda c: f"{c[0]}x{c[1]}x{c[2]}-T{c[3]}-{str(c[4])[6:]}-{'precise' if c[5] else 'default'}")
def test_random_shapes_with_bias_residual_and_precise_intermediate(case):
    # the same with a bias, a residual that aliases the output (every other case) and, for half of the cases, the
    # fp16-times-power-of-two intermediate of bf16 linears switched on
    from nanoquant_b200 import ops
    from nanoquant_b200.kernel import utils as ku
    N, R, M, T, dtype, precise, alias = case
    L = make_layer(N, R, M, T, dtype, seed=N + 5 * R + 11 * M + T)
    g = torch.Generator(device="cuda").manual_seed(N + T)
    scale = float(np.max(np.abs(L["y64"]))) or 1.0
    bias = (torch.randn(M, generator=g, device="cuda") * scale).to(dtype)
    resid = (torch.randn(T, M, generator=g, device="cuda") * scale).to(dtype)
    y64 = L["y64"] + exact_np(bias)[None, :] + exact_np(resid)
    vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
    old = ops.set_precise_intermediate(precise)
    try:
        r = resid.clone()
        layer = (L["s_pre"], vt, L["s_mid"], ut, L["s_post"], R)
        y = ops.group_forward([L["x"]], [layer], T, dtype, L["x"].device, [bias], [r], out=r if alias else None)[0]
        torch.cuda.synchronize()
    finally:
        ops.set_precise_intermediate(old)
    assert y.shape == (T, M)
    assert parity_excess(exact_np(y), y64, dtype) <= 0
