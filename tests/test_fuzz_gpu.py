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
