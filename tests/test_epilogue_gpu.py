"""Bias and residual in the kernels' epilogues (descriptor fields ``bias`` / ``residual``), GEMV and GEMM, both
types, through the C ABI, against the fp64 oracle: ``y = s_out * (U (s_mid * (V (s_in * x)))) + bias + residual``
(the bias add of the reference's PyTorch path, ``src/nanoquant/modules/linear.py:148-149``)."""
import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc
from tests.util import assert_parity, exact_np, make_layer, np_to_torch, tiles_on_gpu

pytestmark = pytest.mark.gpu

DT = {torch.float16: 0, torch.bfloat16: 1}


def run_desc(L, T, dtype, bias, resid, ldr_pad=0, alias=False):
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    N, R, M = L["N"], L["R"], L["M"]
    vt, ut = tiles_on_gpu(L["V"]), tiles_on_gpu(L["U"])
    y = torch.full((T, M), float("nan"), dtype=dtype, device="cuda")
    rbuf = None
    if resid is not None:
        rbuf = torch.zeros(T, M + ldr_pad, dtype=dtype, device="cuda")
        rbuf[:, :M] = resid
        if alias:           # residual read from the output buffer itself (the skip connection updated in place)
            y = rbuf[:, :M]
    d = _lib.LinearDesc(L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                        L["s_post"].data_ptr(), y.data_ptr(), N, R, M, N, y.stride(0),
                        bias.data_ptr() if bias is not None else None,
                        rbuf.data_ptr() if rbuf is not None else None, rbuf.stride(0) if rbuf is not None else 0)
    arr = (_lib.LinearDesc * 1)(d)
    st = torch.cuda.current_stream().cuda_stream
    gemv = T <= Lb.nq_gemv_max_tokens()
    size_fn, fwd = ((Lb.nq_gemv_group_scratch_bytes, Lb.nq_gemv_group_fwd) if gemv
                    else (Lb.nq_gemm_group_scratch_bytes, Lb.nq_gemm_group_fwd))
    nb = size_fn(arr, 1, T)
    scratch = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    _lib.check(fwd(arr, 1, T, DT[dtype], scratch.data_ptr(), nb, st), "fwd")
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    return y, (vt, ut, rbuf)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 3, 7, 40, 200])       # GEMV (1, 3, 7 = two launches), split-K GEMM (40), GEMM (200)
@pytest.mark.parametrize("mode", ["bias", "residual", "both"])
def test_bias_and_residual_vs_oracle(T, dtype, mode):
    N, R, M = 1024, 264, 776          # M not a multiple of 32: ragged last tile in both kernels
    L = make_layer(N, R, M, T, dtype, seed=T + len(mode))
    g = np.random.default_rng(T)
    scale = float(np.abs(L["y64"]).max())
    bias = np_to_torch(g.standard_normal(M) * scale, dtype) if mode != "residual" else None
    resid = np_to_torch(g.standard_normal((T, M)) * scale, dtype) if mode != "bias" else None
    y, keep = run_desc(L, T, dtype, bias, resid, ldr_pad=8)
    y64 = L["y64"].copy()
    if bias is not None:
        y64 = y64 + exact_np(bias)
    if resid is not None:
        y64 = y64 + exact_np(resid)
    assert_parity(exact_np(y), y64, dtype, what=f"T={T} {mode}")
    # without the extra terms the same call reproduces the plain linear
    y0, _ = run_desc(L, T, dtype, None, None)
    assert_parity(exact_np(y0), L["y64"], dtype, what="plain")


@pytest.mark.parametrize("T", [2, 64])
def test_residual_may_alias_the_output(T):
    L = make_layer(512, 96, 256, T, torch.bfloat16, seed=T)
    g = np.random.default_rng(3)
    resid = np_to_torch(g.standard_normal((T, 256)) * float(np.abs(L["y64"]).max()), torch.bfloat16)
    y, keep = run_desc(L, T, torch.bfloat16, None, resid, alias=True)
    assert_parity(exact_np(y), L["y64"] + exact_np(resid), torch.bfloat16, what="in-place skip connection")


def test_module_with_bias_applies_it():
    # a module built with bias=True adds it on both kernel paths (the reference's kernel branches drop it)
    from nanoquant_b200.modules.linear import NanoQuantLinear
    N, R, M = 512, 128, 256
    d = oc.synth_linear(N, R, M, 3, seed=5)
    g = torch.Generator().manual_seed(1)
    bias = (torch.randn(M, generator=g) * 0.01).to(torch.bfloat16)
    for kernel_type, T in (("gemv", 3), ("gemm", 100)):
        m = NanoQuantLinear(N, M, R, has_scale_mid=True, bias=True).cuda()
        with torch.no_grad():
            m.V.copy_(torch.from_numpy(d["V"]).float())
            m.U.copy_(torch.from_numpy(d["U"]).float())
            m.scale_pre.copy_(torch.from_numpy(d["s_pre"]).float()[None])
            m.scale_mid.copy_(torch.from_numpy(d["s_mid"]).float()[None])
            m.scale_post.copy_(torch.from_numpy(d["s_post"]).float()[None])
            m.bias.copy_(bias.float())
        m._prepare_kernel(kernel_type, torch.bfloat16)
        x = torch.randn(T, N, generator=g).to(torch.bfloat16).cuda()
        y = m(x)
        s = lambda a: exact_np(torch.from_numpy(a).float().to(torch.bfloat16))
        y64 = oc.forward_fp64(exact_np(x), d["V"], d["U"], s(d["s_pre"]), s(d["s_mid"]), s(d["s_post"]), bias=exact_np(bias))
        assert_parity(exact_np(y), y64, torch.bfloat16, what=kernel_type)
