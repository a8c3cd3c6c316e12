"""``nq_gemv_group_fwd`` with several linears per launch (the launches a decode step is made of) through the
C ABI: every output against the fp64 oracle on the same seeded inputs, and bit-equal to the same linear run
alone through ``nq_gemv_fwd`` (all accumulation is exact integer arithmetic on a per-token fixed-point image,
so the way rows are dealt to CTAs and launches cannot change a result)."""
import ctypes

import pytest
import torch

from tests.util import assert_parity, exact_np, make_group, tiles_on_gpu

pytestmark = pytest.mark.gpu

DT = {torch.float16: 0, torch.bfloat16: 1}


def run_group(layers, T, dtype, pad=0, bias=None, residual=None):
    """One group launch with the outputs side by side in one [T, sum(M) + pad] buffer (ldy > M); returns the
    per-linear output views, the descriptors and the tensors that must stay alive."""
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    width = sum(L["M"] for L in layers) + pad
    ybuf = torch.full((T, width), float("nan"), dtype=dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    keep, descs, col = [], [], 0
    for L in layers:
        vt, ut = tiles_on_gpu(L["V"]), tiles_on_gpu(L["U"])
        keep += [vt, ut]
        descs.append(_lib.LinearDesc(L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(),
                                     L["s_mid"].data_ptr() if L["s_mid"] is not None else None, ut.data_ptr(),
                                     L["s_post"].data_ptr(), ybuf.data_ptr() + 2 * col, L["N"], L["R"], L["M"],
                                     L["x"].stride(0), width))
        col += L["M"]
    arr = (_lib.LinearDesc * len(descs))(*descs)
    nbytes = Lb.nq_gemv_group_scratch_bytes(arr, len(descs), T)
    assert nbytes > 0
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for _ in range(2):   # the second launch on the same scratch finds the first one's tagged intermediate
        _lib.check(Lb.nq_gemv_group_fwd(arr, len(descs), T, DT[dtype], scratch.data_ptr(), nbytes, st), "group")
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    outs, col = [], 0
    for L in layers:
        outs.append(ybuf[:, col:col + L["M"]])
        col += L["M"]
    if pad:
        assert torch.isnan(ybuf[:, col:]).all()          # nothing is written beyond the last linear
    return outs, descs, keep


def run_single(L, d, T, dtype):
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    nb = Lb.nq_gemv_scratch_bytes(T, L["N"], L["R"], L["M"])
    s1 = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    y1 = torch.empty(T, L["M"], dtype=dtype, device="cuda")
    x = L["x"].contiguous()
    _lib.check(Lb.nq_gemv_fwd(x.data_ptr(), d.s_in, d.v_tiles, d.s_mid, d.u_tiles, d.s_out, y1.data_ptr(),
                              s1.data_ptr(), nb, T, L["N"], L["R"], L["M"], DT[dtype], st), "single")
    assert Lb.nq_scratch_status(s1.data_ptr(), st) == 0
    return y1


def check_group(shapes, T, dtype, seed, no_mid=(), pad=0):
    layers = make_group(shapes, T, dtype, seed=seed, no_mid=no_mid)
    outs, descs, keep = run_group(layers, T, dtype, pad=pad)
    for i, (L, y, d) in enumerate(zip(layers, outs, descs)):
        assert_parity(exact_np(y), L["y64"], dtype, what=f"linear {i} of {shapes}")
        assert torch.equal(y, run_single(L, d, T, dtype)), f"linear {i}: group launch differs from the single launch"


# launch groups of the workloads: (N, R, M) per linear, ranks from the reference's rank formula
QWEN3_QKV = [(4096, 1600, 4096), (4096, 608, 1024), (4096, 608, 1024)]
QWEN3_GATE_UP = [(4096, 2432, 12288)] * 2          # 768 row tiles over 148 CTAs: one CTA's range crosses the job boundary
LLAMA1B_QKV = [(2048, 992, 2048), (2048, 384, 512), (2048, 384, 512)]   # 36 phase-1 tiles: most CTAs own no tile
LLAMA1B_GATE_UP = [(2048, 1600, 8192)] * 2
L70B_QKV_SHARD = [(8192, 3232, 1024), (8192, 704, 128), (8192, 704, 128)]   # U split eight ways by output rows
L70B_GATE_UP_SHARD = [(8192, 5056, 3584)] * 2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 2, 4])
@pytest.mark.parametrize("shapes", [QWEN3_QKV, QWEN3_GATE_UP], ids=["qkv", "gate_up"])
def test_qwen3_8b_groups(shapes, T, dtype):
    check_group(shapes, T, dtype, seed=100 + T)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shapes", [LLAMA1B_QKV, LLAMA1B_GATE_UP], ids=["qkv", "gate_up"])
def test_llama_1b_groups(shapes, dtype):
    check_group(shapes, 1, dtype, seed=7)
    check_group(shapes, 4, dtype, seed=8)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shapes", [L70B_QKV_SHARD, L70B_GATE_UP_SHARD], ids=["qkv", "gate_up"])
def test_llama_70b_shard_groups(shapes, dtype):
    check_group(shapes, 1, dtype, seed=9)
    check_group(shapes, 2, dtype, seed=10)


@pytest.mark.parametrize("T", [1, 3, 4, 7])
def test_four_ragged_linears_one_without_middle_scale(T):
    # four linears, ragged widths (not multiples of 32, 16 or 8), different ranks, one without s_mid,
    # padding columns behind the last output; T = 7 runs as two launches on the same scratch
    shapes = [(1000, 136, 300), (1000, 72, 17), (1000, 264, 1001), (1000, 32, 40)]
    check_group(shapes, T, torch.float16, seed=20 + T, no_mid=(2,), pad=5)


def test_group_of_linears_with_different_inputs():
    # the linears of a group need not share their input (nor its width)
    shapes = [(512, 128, 256), (768, 96, 64)]
    check_group(shapes, 2, torch.bfloat16, seed=31)


def test_single_qwen3_projections_at_decode_batches():
    # q/o (R = 1600) and down alone, batches 1 and 4, both types
    for (N, R, M) in [(4096, 1600, 4096), (12288, 2432, 4096)]:
        for dtype in (torch.float16, torch.bfloat16):
            check_group([(N, R, M)], 4, dtype, seed=N + R)
            check_group([(N, R, M)], 1, dtype, seed=N + R + 1)
