"""Prefill GEMM (tcgen05) through the reference's Marlin-layout operators and through the C ABI,
against the fp64 oracle on the same seeded inputs."""
import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc
from tests.util import parity_excess, TOL, exact_np, half2_bits, make_layer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    import binary_kernels  # noqa: F401
    return torch.ops.binary_kernels


def marlin_operands(L, dtype):
    """Operands exactly as the reference's fused Marlin packer lays them out (numpy oracle of it)."""
    npdt = np.float16
    to_np = lambda t: t.float().cpu().numpy().astype(np.float32)
    # permutations act on positions only: run them on float32 copies and convert back
    Vb, Ub, s1, s2, s3, ws = oc.pack_marlin_fused(np.ascontiguousarray(L["V"].T), np.ascontiguousarray(L["U"].T),
                                                   to_np(L["s_pre"]), to_np(L["s_mid"]), to_np(L["s_post"]))
    dev = L["x"].device
    t = lambda a, d=dtype: torch.from_numpy(np.ascontiguousarray(a)).to(d).to(dev)
    return (t(Vb, torch.int32), t(Ub, torch.int32), t(s1), t(s2), t(s3), t(ws, torch.int32))


SHAPES = [
    (4096, 1536, 4096, 128),    # 4096 -> 4096, r = 1536, 128 tokens
    (4096, 608, 1024, 200),     # rank padded to 768 by the Marlin packer, ragged token count
    (4096, 2432, 12288, 512),
    (12288, 2432, 4096, 77),
    (4096, 2944, 11008, 256),   # a shape the reference's Marlin kernel rejects (11008 % 512 != 0)
    (2048, 992, 2048, 2048),
    (4096, 1600, 4096, 16),     # few tokens, few output tiles: the k dimension is split over the idle SMs
    (1024, 288, 576, 33),       # split with a ragged token count and a partial last output tile
    (12288, 2432, 4096, 9),
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", SHAPES)
def test_marlin_nanoquant_forward_vs_oracle(ops, shape, dtype):
    N, R, M, T = shape
    L = make_layer(N, R, M, T, dtype, seed=N + R + T)
    Vb, Ub, s1, s2, s3, ws = marlin_operands(L, dtype)
    y = ops.marlin_nanoquant_forward(L["x"], Vb, Ub, s1, s2, s3, ws)
    assert y.shape == (T, M) and y.dtype == dtype
    assert parity_excess(exact_np(y), L["y64"], dtype) <= 0
    assert torch.equal(y, ops.marlin_nanoquant_forward(L["x"], Vb, Ub, s1, s2, s3, ws))   # deterministic


# shapes of the workloads at their own token counts (the oracle's dense fp64 matmuls take a few seconds each)
CONFIG_CASES = [
    (4096, 2016, 4096, 2048, torch.bfloat16),     # Llama-2-7B q/k/v/o, 1.0 bpw, 2048 tokens
    (4096, 2944, 11008, 2048, torch.bfloat16),    # Llama-2-7B gate/up: 11008 rows, a shape the reference's kernel rejects
    (11008, 2944, 4096, 512, torch.bfloat16),     # Llama-2-7B down
    (8192, 5056, 3584, 512, torch.bfloat16),      # Llama-3-70B gate/up shard (U split eight ways), prefill 512 tokens
    (8192, 3232, 1024, 16, torch.bfloat16),       # Llama-3-70B q shard, decode batch 16
    (4096, 2432, 12288, 16, torch.bfloat16),      # Qwen3-8B gate/up, decode batch 16 (split-K)
    (12288, 2432, 4096, 16, torch.bfloat16),      # Qwen3-8B down, decode batch 16
    (4096, 608, 1024, 16, torch.float16),         # Qwen3-8B k/v, decode batch 16
]


@pytest.mark.parametrize("case", CONFIG_CASES, ids=lambda c: f"{c[0]}-{c[1]}-{c[2]}x{c[3]}")
def test_workload_shapes_at_their_token_counts(case):
    from nanoquant_b200 import ops as nq_ops
    from tests.util import tiles_on_gpu
    N, R, M, T, dtype = case
    L = make_layer(N, R, M, T, dtype, seed=N + M + T)
    y = nq_ops.linear_forward(L["x"], L["s_pre"], tiles_on_gpu(L["V"]), L["s_mid"], tiles_on_gpu(L["U"]), L["s_post"], R)
    assert parity_excess(exact_np(y), L["y64"], dtype) <= 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_marlin_onebit_forward_vs_oracle(ops, dtype):
    # one stage: y = s_out * (W . (s_in * x)), W [n, k]
    n, k, T = 1024, 2048, 300
    g = np.random.default_rng(5)
    W = (g.integers(0, 2, size=(n, k), dtype=np.int8) * 2 - 1).astype(np.int8)
    dev = "cuda"
    s_in = ((torch.rand(k) + 0.5) * 0.01).to(dtype).to(dev)
    s_out = ((torch.rand(n) + 0.5) * 0.01).to(dtype).to(dev)
    x = torch.randn(T, k).to(dtype).to(dev)
    B, si, so, wsz = oc.pack_marlin(W, s_in.float().cpu().numpy(), s_out.float().cpu().numpy())
    t = lambda a, d=dtype: torch.from_numpy(np.ascontiguousarray(a)).to(d).to(dev)
    ws = torch.zeros(wsz, dtype=torch.int32, device=dev)
    y64 = ((exact_np(x) * exact_np(s_in)) @ W.astype(np.float64).T) * exact_np(s_out)
    y = ops.marlin_onebit_forward(x, t(B, torch.int32), t(si), t(so), ws)
    assert parity_excess(exact_np(y), y64, dtype) <= 0
    # optional scales
    y2 = ops.marlin_onebit_forward(x, t(B, torch.int32), None, None, ws)
    y64b = exact_np(x) @ W.astype(np.float64).T
    assert parity_excess(exact_np(y2), y64b, dtype) <= 0


def test_marlin_error_behaviour(ops):
    L = make_layer(256, 256, 128, 16, torch.float16, seed=1)
    Vb, Ub, s1, s2, s3, ws = marlin_operands(L, torch.float16)
    with pytest.raises(RuntimeError, match="k dimension mismatch"):
        ops.marlin_nanoquant_forward(L["x"][:, :128].contiguous(), Vb, Ub, s1, s2, s3, ws)
    with pytest.raises(RuntimeError, match="s_in size mismatch"):
        ops.marlin_nanoquant_forward(L["x"], Vb, Ub, s1[:128].contiguous(), s2, s3, ws)
    with pytest.raises(RuntimeError, match="workspace too small"):
        ops.marlin_nanoquant_forward(L["x"], Vb, Ub, s1, s2, s3, ws[:1])
    with pytest.raises(RuntimeError, match="Half and BFloat16"):
        ops.marlin_nanoquant_forward(L["x"].float(), Vb, Ub, s1, s2, s3, ws)


def test_gemv_op_routes_many_tokens_to_the_gemm(ops):
    L = make_layer(2048, 512, 1024, 130, torch.float16, seed=3)
    y = ops.nanoquant_dyn_forward(L["x"], L["s_pre"], half2_bits(L["V"]), L["s_mid"], half2_bits(L["U"]),
                                  L["s_post"], num_acc_stage1=1, num_acc_stage2=1)
    assert parity_excess(exact_np(y), L["y64"], torch.float16) <= 0


def test_c_abi_gemm_and_gemv_agree_at_the_dispatch_boundary():
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    Lb = _lib.lib()
    N, R, M = 1024, 256, 512
    T = Lb.nq_gemv_max_tokens()
    L = make_layer(N, R, M, T, torch.float16, seed=9)
    vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for fn, nbytes in ((Lb.nq_gemv_fwd, Lb.nq_gemv_scratch_bytes(T, N, R, M)),
                       (Lb.nq_gemm_fwd, Lb.nq_gemm_scratch_bytes(T, N, R, M))):
        scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        y = torch.empty(T, M, dtype=torch.float16, device="cuda")
        _lib.check(fn(L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                      L["s_post"].data_ptr(), y.data_ptr(), scratch.data_ptr(), nbytes, T, N, R, M, _lib.NQ_F16, st),
                   "fwd")
        assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
        outs.append(y)
        assert parity_excess(exact_np(y), L["y64"], torch.float16) <= 0
    # two different arithmetic paths, both inside the bar: they agree to twice the bar
    assert oc.rel_err(exact_np(outs[0]), exact_np(outs[1])) <= 2 * TOL[torch.float16]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1032, 264, 1001, 7), (4096, 1608, 4099, 23), (520, 8, 33, 64)])
def test_c_abi_linear_few_tokens_ragged_split(shape, dtype):
    # 5..64 tokens: nq_linear_fwd takes the GEMM with the k dimension split over CTAs.  Ragged rank, output
    # width (odd: element stores) and token count; the scratch is shared with a decode call in between, which
    # must leave the tile counters in the header alone; the result is the same bit for bit on every call.
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    Lb = _lib.lib()
    N, R, M, T = shape
    L = make_layer(N, R, M, T, dtype, seed=sum(shape))
    vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
    ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
    st = torch.cuda.current_stream().cuda_stream
    dt = _lib.NQ_F16 if dtype == torch.float16 else _lib.NQ_BF16
    nbytes = max(Lb.nq_linear_scratch_bytes(T, N, R, M), Lb.nq_linear_scratch_bytes(1, N, R, M))
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    args = lambda x, y, t: (x.data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                            L["s_post"].data_ptr(), y.data_ptr(), scratch.data_ptr(), nbytes, t, N, R, M, dt, st)
    ys = []
    for rep in range(3):
        y = torch.empty(T, M, dtype=dtype, device="cuda")
        _lib.check(Lb.nq_linear_fwd(*args(L["x"], y, T)), "nq_linear_fwd")
        ys.append(y)
        if rep == 0:   # a one-token decode call on the same scratch between two GEMM calls
            y1 = torch.empty(1, M, dtype=dtype, device="cuda")
            _lib.check(Lb.nq_linear_fwd(*args(L["x"][:1].contiguous(), y1, 1)), "nq_linear_fwd")
            assert oc.rel_err(exact_np(y1), L["y64"][:1]) <= 2 * TOL[dtype]
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    assert parity_excess(exact_np(ys[0]), L["y64"], dtype) <= 0
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[1], ys[2])


@pytest.mark.parametrize("T", [6, 16, 300])
def test_c_abi_gemm_group_matches_single_linears(T):
    # q/k/v-like group (shared input, different ranks and widths) in one launch per stage against the oracle and
    # against the per-linear entry point; outputs written side by side into one buffer (ldy > M)
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    Lb = _lib.lib()
    N = 1024
    shapes = [(N, 264, 1024), (N, 96, 256), (N, 96, 384)]
    layers = [make_layer(n, r, m, T, torch.bfloat16, seed=10 + i) for i, (n, r, m) in enumerate(shapes)]
    x = layers[0]["x"]
    for L in layers[1:]:   # the same activations for the whole group: recompute the oracle on them
        L["x"] = x
        L["y64"] = oc.forward_fp64(exact_np(x), L["V"], L["U"], exact_np(L["s_pre"]), exact_np(L["s_mid"]), exact_np(L["s_post"]))
    width = sum(m for (_, _, m) in shapes)
    ybuf = torch.zeros(T, width, dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    keep, descs, col = [], [], 0
    for L, (n, r, m) in zip(layers, shapes):
        vt = ku.pack_tiles(half2_bits(L["V"]), (r, n), "half2")
        ut = ku.pack_tiles(half2_bits(L["U"]), (m, r), "half2")
        keep += [vt, ut]
        descs.append(_lib.LinearDesc(x.data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                                     L["s_post"].data_ptr(), ybuf.data_ptr() + 2 * col, n, r, m, n, width))
        col += m
    arr = (_lib.LinearDesc * len(descs))(*descs)
    nbytes = Lb.nq_gemm_group_scratch_bytes(arr, len(descs), T)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    for _ in range(2):
        _lib.check(Lb.nq_gemm_group_fwd(arr, len(descs), T, _lib.NQ_BF16, scratch.data_ptr(), nbytes, st), "group")
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    col = 0
    for L, (n, r, m), d in zip(layers, shapes, descs):
        y = ybuf[:, col:col + m]
        assert parity_excess(exact_np(y), L["y64"], torch.bfloat16) <= 0
        y1 = torch.empty(T, m, dtype=torch.bfloat16, device="cuda")
        nb1 = Lb.nq_gemm_scratch_bytes(T, n, r, m)
        s1 = torch.zeros(nb1, dtype=torch.uint8, device="cuda")
        _lib.check(Lb.nq_gemm_fwd(x.data_ptr(), d.s_in, d.v_tiles, d.s_mid, d.u_tiles, d.s_out, y1.data_ptr(),
                                  s1.data_ptr(), nb1, T, n, r, m, _lib.NQ_BF16, st), "single")
        assert oc.rel_err(exact_np(y), exact_np(y1)) <= 2.0 ** -7   # same products, possibly another k split
        col += m


@pytest.fixture
def precise_intermediate():
    from nanoquant_b200 import ops
    old = ops.set_precise_intermediate(True)
    yield
    ops.set_precise_intermediate(old)


@pytest.mark.parametrize("T,N,R,M", [(7, 1032, 264, 1001), (16, 4096, 1600, 4096), (128, 4096, 1536, 4096), (300, 2048, 1000, 1536),
                                     (2048, 2048, 1024, 2048)])
def test_precise_intermediate_of_bf16_linears(precise_intermediate, T, N, R, M):
    # The rank-R intermediate as fp16 times a per-token power of two (slab split, cluster split and plain tiles):
    # inside the parity bar like the default, and the error BEYOND the output's own rounding is below 1e-3 of the
    # maximum (with the bf16 intermediate it is up to 1.6e-3).  A token scaled by 2^20 and one by 2^-20 check that
    # the exponents follow the tokens, and an all-zero token that nothing divides by zero.
    from nanoquant_b200 import _lib
    from tests.util import tiles_on_gpu, elementwise_bound
    Lb = _lib.lib()
    dtype = torch.bfloat16
    L = make_layer(N, R, M, T, dtype, seed=40 + T)
    x = L["x"].clone()
    if T >= 7:
        x[1] *= 2.0 ** 20
        x[2] *= 2.0 ** -20
        x[3] = 0
    y64 = oc.forward_fp64(exact_np(x), L["V"], L["U"], exact_np(L["s_pre"]), exact_np(L["s_mid"]), exact_np(L["s_post"]))
    vt, ut = tiles_on_gpu(L["V"]), tiles_on_gpu(L["U"])
    y = torch.full((T, M), float("nan"), dtype=dtype, device="cuda")
    nb = Lb.nq_gemm_scratch_bytes(T, N, R, M)
    scratch = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        _lib.check(Lb.nq_gemm_fwd(x.data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                                  L["s_post"].data_ptr(), y.data_ptr(), scratch.data_ptr(), nb, T, N, R, M, _lib.NQ_BF16, st), "gemm")
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    yn = exact_np(y)
    for rows in ([1], [2], [3], [r for r in range(T) if r not in (1, 2, 3)] if T >= 7 else list(range(T))):
        if T < 7 and rows != list(range(T)):
            continue
        a, b = yn[rows], y64[rows]
        if not np.any(b):
            assert not np.any(a)
            continue
        half_ulp = elementwise_bound(b, dtype, 0.0, a)
        beyond = np.max(np.abs(a - b) - half_ulp) / np.max(np.abs(b))
        assert beyond <= 1e-3, (rows[:3], beyond)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T", [25, 40, 100, 128, 200, 300])
def test_c_abi_gemm_cluster_split(T, dtype):
    # Few output tiles above 24 tokens: the k dimension is split over the CTAs of a thread-block cluster, which add
    # their partial sums through distributed shared memory.  Two linears with different ranks in one launch, so the
    # chunks per CTA differ per job and the last CTA of a cluster has no chunk of the smaller job (it contributes
    # zeros); ragged token counts; the result must not change from run to run (fixed summation order).
    from nanoquant_b200 import _lib
    from tests.util import make_group, tiles_on_gpu, assert_parity
    Lb = _lib.lib()
    code = _lib.NQ_BF16 if dtype == torch.bfloat16 else _lib.NQ_F16
    shapes = [(1024, 1288, 256), (1024, 2048, 200)]
    layers = make_group(shapes, T, dtype, seed=300 + T)
    width = 512
    ybuf = torch.zeros(T, width, dtype=dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    keep, descs = [], []
    for i, (L, (n, r, m)) in enumerate(zip(layers, shapes)):
        vt, ut = tiles_on_gpu(L["V"]), tiles_on_gpu(L["U"])
        keep += [vt, ut]
        descs.append(_lib.LinearDesc(L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
                                     L["s_post"].data_ptr(), ybuf.data_ptr() + 2 * 256 * i, n, r, m, n, width))
    arr = (_lib.LinearDesc * len(descs))(*descs)
    nbytes = Lb.nq_gemm_group_scratch_bytes(arr, len(descs), T)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    outs = []
    for _ in range(3):
        ybuf.fill_(7.0)
        _lib.check(Lb.nq_gemm_group_fwd(arr, len(descs), T, code, scratch.data_ptr(), nbytes, st), "group")
        outs.append(ybuf.clone())
    assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    for i, (L, (n, r, m)) in enumerate(zip(layers, shapes)):
        assert_parity(exact_np(ybuf[:, 256 * i:256 * i + m]), L["y64"], dtype)
    assert torch.all(ybuf[:, 256 + 200:] == 7.0)   # columns beyond the second linear's width are untouched


def test_gemm_linearity_full_size(ops):
    # size-independent property at a full-size shape: the op is linear in x.  Doubling x doubles every
    # fp32 partial sum exactly; only intermediate values that fall into the fp16 subnormal range may
    # round differently, so the two results agree to well below the parity bar, not bit for bit.
    L = make_layer(4096, 1600, 4096, 256, torch.float16, seed=11)
    Vb, Ub, s1, s2, s3, ws = marlin_operands(L, torch.float16)
    s2, s3 = s2 * 64, s3 * 16
    y = ops.marlin_nanoquant_forward(L["x"], Vb, Ub, s1, s2, s3, ws)
    y2 = ops.marlin_nanoquant_forward(L["x"] * 2, Vb, Ub, s1, s2, s3, ws)
    assert oc.rel_err(exact_np(y2), 2 * exact_np(y)) <= 2e-4
    assert float((y2 == y * 2).float().mean()) > 0.99


def test_module_kernel_paths():
    from nanoquant_b200.modules.linear import NanoQuantLinear
    N, R, M = 512, 128, 256
    d = oc.synth_linear(N, R, M, 3, seed=21)
    for kernel_type, T in (("gemv", 3), ("gemm", 160)):
        m = NanoQuantLinear(N, M, R, has_scale_mid=True).cuda()
        with torch.no_grad():
            m.V.copy_(torch.from_numpy(d["V"]).float())
            m.U.copy_(torch.from_numpy(d["U"]).float())
            m.scale_pre.copy_(torch.from_numpy(d["s_pre"]).float()[None])
            m.scale_mid.copy_(torch.from_numpy(d["s_mid"]).float()[None])
            m.scale_post.copy_(torch.from_numpy(d["s_post"]).float()[None])
        with pytest.raises(RuntimeError, match="_prepare_kernel"):
            m(torch.zeros(1, N, device="cuda"))
        sd = m.state_dict()
        assert np.array_equal(sd["V_packed"].cpu().numpy(), oc.pack_rows(d["V"], "lsb_first"))
        assert tuple(sd["U_shape"].tolist()) == (M, R)
        # the module keeps its scales in bf16 (like the reference); compare with those exact values
        sp, sm, so = (exact_np(m.scale_pre)[0], exact_np(m.scale_mid)[0], exact_np(m.scale_post)[0])
        m._prepare_kernel(kernel_type, torch.bfloat16)
        x = torch.randn(2, T // 2 if T > 3 else 1, N, device="cuda").to(torch.bfloat16)
        if T == 3:
            x = torch.randn(3, N, device="cuda").to(torch.bfloat16)
        y = m(x)
        y64 = oc.forward_fp64(exact_np(x).reshape(-1, N), d["V"], d["U"], sp, sm, so)
        assert y.shape[:-1] == x.shape[:-1] and y.shape[-1] == M
        assert parity_excess(exact_np(y).reshape(-1, M), y64, torch.bfloat16) <= 0


def test_module_fold_input_scale():
    """A per-column weight folded into scale_pre (the RMSNorm weight in front of the linear) equals scaling x."""
    from nanoquant_b200.modules.linear import NanoQuantLinear
    N, R, M, T = 512, 160, 384, 3
    d = oc.synth_linear(N, R, M, T, seed=8)
    tt = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    g = torch.Generator().manual_seed(1)
    w = (torch.rand(N, generator=g) + 0.5).to(torch.float16)
    for kernel_type in ("gemv", "gemm"):
        m = NanoQuantLinear(N, M, R, has_scale_mid=True).cuda()
        with torch.no_grad():
            m.V.copy_(tt(d["V"]).float())
            m.U.copy_(tt(d["U"]).float())
            m.scale_pre.copy_(tt(d["s_pre"]).float()[None])
            m.scale_mid.copy_(tt(d["s_mid"]).float()[None])
            m.scale_post.copy_(tt(d["s_post"]).float()[None])
        m.fold_input_scale(w)
        sp, sm, so = (exact_np(m.scale_pre)[0], exact_np(m.scale_mid)[0], exact_np(m.scale_post)[0])
        # the folded scale is the product rounded once to the module's dtype
        want = (tt(d["s_pre"]).to(torch.bfloat16).float() * w.float()).to(torch.bfloat16)
        assert torch.equal(m.scale_pre.detach().cpu()[0], want)
        m._prepare_kernel(kernel_type, torch.float16)
        x = tt(d["x"]).cuda()
        y64 = oc.forward_fp64(d["x"], d["V"], d["U"], sp, sm, so)
        assert parity_excess(exact_np(m(x)), y64, torch.float16) <= 0
        # folding works after the layer has been prepared as well (the input scale then is `scale_pre` / `s1`)
        ones = torch.full((N,), 2.0, dtype=torch.float16)
        m.fold_input_scale(ones)
        assert parity_excess(exact_np(m(x)), 2 * y64, torch.float16) <= 0
    with pytest.raises(ValueError):
        m2 = NanoQuantLinear(N, M, R)
        m2.fold_input_scale(w[:-1])


def test_module_load_packed_checkpoint_tensors():
    from nanoquant_b200.modules.linear import NanoQuantLinear
    N, R, M, T = 512, 160, 384, 2
    d = oc.synth_linear(N, R, M, T, seed=4)
    m = NanoQuantLinear(N, M, R, has_scale_mid=True)
    tt = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    m.load_packed(tt(oc.pack_rows(d["V"], "lsb_first")), (R, N), tt(oc.pack_rows(d["U"], "lsb_first")), (M, R),
                  tt(d["s_pre"])[None], tt(d["s_post"])[None], tt(d["s_mid"])[None], dtype=torch.float16)
    x = tt(d["x"]).cuda()
    y = m(x)
    y64 = oc.forward_fp64(d["x"], d["V"], d["U"], d["s_pre"], d["s_mid"], d["s_post"])
    assert parity_excess(exact_np(y), y64, torch.float16) <= 0
