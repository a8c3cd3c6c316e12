"""Decode GEMV through ``torch.ops.binary_kernels.nanoquant_dyn_forward`` (which
calls the C ABI) against the fp64 oracle on the same seeded inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc
from tests.util import parity_excess, TOL, exact_np, half2_bits, make_layer, np_to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def op():
    import binary_kernels  # noqa: F401
    return torch.ops.binary_kernels.nanoquant_dyn_forward


KW = dict(num_acc_stage1=1, num_acc_stage2=1)


def run(op, L):
    return op(L["x"], L["s_pre"], half2_bits(L["V"]), L["s_mid"], half2_bits(L["U"]), L["s_post"], **KW)


def test_golden_forward_fp64(op, golden_dir):
    g = np.load(os.path.join(golden_dir, "forward_fp64.npz"))
    for name in "abc":
        s_mid = np_to_torch(g[f"{name}_s_mid"], torch.float16) if f"{name}_s_mid" in g else None
        y = op(np_to_torch(g[f"{name}_x"], torch.float16), np_to_torch(g[f"{name}_s_pre"], torch.float16),
               half2_bits(g[f"{name}_V"]), s_mid, half2_bits(g[f"{name}_U"]),
               np_to_torch(g[f"{name}_s_post"], torch.float16), **KW)
        assert parity_excess(exact_np(y), g[f"{name}_y"], torch.float16) <= 0, name


SHAPES = [
    (4096, 1536, 4096, 1),     # 4096 -> 4096, r = 1536, one token
    (4096, 1536, 4096, 4),
    (4096, 608, 1024, 1),      # Qwen3-8B k/v projection
    (4096, 2432, 12288, 2),    # gate / up
    (12288, 2432, 4096, 3),    # down
    (2048, 992, 2048, 1),      # Llama-3.2-1B q/o
    (160, 64, 40, 1),          # ragged: K not a multiple of 256, rows not of 32
    (96, 32, 17, 4),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemv_vs_oracle(op, shape, dtype):
    N, R, M, T = shape
    L = make_layer(N, R, M, T, dtype, seed=N + R + M + T)
    y = run(op, L)
    assert y.shape == (T, M) and y.dtype == dtype
    assert parity_excess(exact_np(y), L["y64"], dtype) <= 0


@pytest.mark.parametrize("T", [5, 8, 16])
def test_gemv_more_than_four_tokens(op, T):
    L = make_layer(1024, 320, 768, T, torch.float16, seed=T)
    assert parity_excess(exact_np(run(op, L)), L["y64"], torch.float16) <= 0


@pytest.mark.parametrize("T", [5, 9])
def test_c_abi_gemv_more_tokens_than_one_launch(T):
    # nq_gemv_fwd itself (not the dispatcher) with more tokens than one launch takes: several launches of
    # up to four tokens on the same scratch
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    Lb = _lib.lib()
    N, R, M = 1000, 136, 300      # unaligned input rows (N % 8 != 0 is fine for the GEMV), ragged rank and width
    L = make_layer(N, R, M, T, torch.float16, seed=T)
    vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
    st = torch.cuda.current_stream().cuda_stream
    nbytes = Lb.nq_gemv_scratch_bytes(T, N, R, M)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    y = torch.empty(T, M, dtype=torch.float16, device="cuda")
    _lib.check(Lb.nq_gemv_fwd(L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(),
                              ut.data_ptr(), L["s_post"].data_ptr(), y.data_ptr(), scratch.data_ptr(), nbytes,
                              T, N, R, M, _lib.NQ_F16, st), "nq_gemv_fwd")
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    assert parity_excess(exact_np(y), L["y64"], torch.float16) <= 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8192, 5056, 3584, 2), (28672, 5056, 1024, 1), (28672, 5056, 1024, 4)])
def test_gemv_70b_shard_shapes(op, shape, dtype):
    # Llama-3-70B-shaped gate/up and down projections at 0.8 bpw with U split eight ways by output rows
    N, R, M, T = shape
    L = make_layer(N, R, M, T, dtype, seed=N + M)
    assert parity_excess(exact_np(run(op, L)), L["y64"], dtype) <= 0


@pytest.mark.parametrize("T", [1, 4])
@pytest.mark.parametrize("shape", [(2048, 384, 512), (2048, 1600, 8192), (8192, 1600, 2048)])
def test_gemv_llama_1b_shapes(op, shape, T):
    # Llama-3.2-1B k/v, gate/up and down at 1.0 bpw in the type the decode workload runs in
    N, R, M = shape
    L = make_layer(N, R, M, T, torch.bfloat16, seed=N + R + T)
    assert parity_excess(exact_np(run(op, L)), L["y64"], torch.bfloat16) <= 0


def test_gemv_without_scale_mid_and_1d_input(op):
    L = make_layer(512, 128, 256, 1, torch.float16, seed=2, has_mid=False)
    y2 = run(op, L)
    L1 = dict(L, x=L["x"][0])
    y1 = run(op, L1)
    assert y1.shape == (256,)
    assert torch.equal(y1, y2[0])
    assert parity_excess(exact_np(y2), L["y64"], torch.float16) <= 0


def test_gemv_is_deterministic_and_token_independent(op):
    L = make_layer(2048, 512, 1024, 4, torch.float16, seed=7)
    y = run(op, L)
    assert torch.equal(y, run(op, L))
    # a token computed alone equals the same token computed in a batch: the fixed-point scale is per token
    for t in range(4):
        Lt = dict(L, x=L["x"][t:t + 1].contiguous())
        assert torch.equal(run(op, Lt)[0], y[t])


def test_gemv_linearity_in_scales(op):
    # doubling s_post doubles y exactly (power-of-two scaling commutes with every rounding step)
    # (outputs are kept well inside the fp16 normal range so that the doubling itself is exact)
    L = make_layer(1024, 256, 512, 2, torch.float16, seed=3)
    L = dict(L, s_post=(L["s_post"] * 1024))
    y = run(op, L)
    assert float(y.abs().min()) == 0.0 or float(y.abs()[y != 0].min()) > 6.2e-5
    L2 = dict(L, s_post=(L["s_post"] * 2))
    assert torch.equal(run(op, L2), y * 2)


def test_gemv_tiles_operands_equal_half2_operands(op):
    from nanoquant_b200.kernel import utils as ku
    L = make_layer(1024, 288, 640, 3, torch.bfloat16, seed=5)
    y = run(op, L)
    vt = ku.pack_tiles(half2_bits(L["V"]), (288, 1024), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (640, 288), "half2")
    y2 = op(L["x"], L["s_pre"], vt, L["s_mid"], ut, L["s_post"], **KW)
    assert torch.equal(y, y2)


def test_gemv_zero_and_extreme_inputs(op):
    L = make_layer(512, 128, 256, 2, torch.float16, seed=4)
    L0 = dict(L, x=torch.zeros_like(L["x"]))
    assert torch.count_nonzero(run(op, L0)) == 0
    # fp16 saturation bound of the reference epilogue
    Lbig = dict(L, x=L["x"] * 0 + 60000, s_pre=L["s_pre"] * 0 + 1, s_mid=L["s_mid"] * 0 + 1,
                s_post=L["s_post"] * 0 + 1, V=np.ones_like(L["V"]), U=np.ones_like(L["U"]))
    y = run(op, Lbig)
    assert torch.all(y == 64504.0) or torch.all(y.float() == torch.tensor(64504.0).half().float())


def test_gemv_error_behaviour(op):
    L = make_layer(256, 64, 128, 1, torch.float16, seed=1)
    vb, ub = half2_bits(L["V"]), half2_bits(L["U"])
    with pytest.raises(ValueError, match="n_acc1 should be one of"):
        op(L["x"], L["s_pre"], vb, L["s_mid"], ub, L["s_post"])          # schema default num_acc=4
    with pytest.raises(RuntimeError, match="Half or BFloat16"):
        op(L["x"].float(), L["s_pre"], vb, L["s_mid"], ub, L["s_post"], **KW)
    with pytest.raises(RuntimeError, match="scale_l size mismatch"):
        op(L["x"], L["s_pre"], vb, L["s_mid"][:32].contiguous(), ub, L["s_post"], **KW)
    with pytest.raises(RuntimeError, match="contiguous"):
        op(L["x"], L["s_pre"], vb.t().contiguous().t(), L["s_mid"], ub, L["s_post"], **KW)
    with pytest.raises(RuntimeError, match="int32"):
        op(L["x"], L["s_pre"], vb.to(torch.int64), L["s_mid"], ub, L["s_post"], **KW)


def test_fake_impl_and_graph_capture(op):
    L = make_layer(1024, 256, 512, 1, torch.bfloat16, seed=9)
    vb, ub = half2_bits(L["V"]), half2_bits(L["U"])
    with torch._subclasses.FakeTensorMode():
        fx = torch.empty(3, 1024, dtype=torch.bfloat16, device="cuda")
        fy = op(fx, torch.empty(1024, dtype=torch.bfloat16, device="cuda"),
                torch.empty(256, 32, dtype=torch.int32, device="cuda"), None,
                torch.empty(512, 8, dtype=torch.int32, device="cuda"),
                torch.empty(512, dtype=torch.bfloat16, device="cuda"), **KW)
        assert fy.shape == (3, 512) and fy.dtype == torch.bfloat16
    y_eager = op(L["x"], L["s_pre"], vb, L["s_mid"], ub, L["s_post"], **KW)   # also builds the tile cache
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        y_warm = op(L["x"], L["s_pre"], vb, L["s_mid"], ub, L["s_post"], **KW)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            y_graph = op(L["x"], L["s_pre"], vb, L["s_mid"], ub, L["s_post"], **KW)
        g.replay()
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_graph, y_eager) and torch.equal(y_warm, y_eager)
