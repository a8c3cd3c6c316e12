"""Parity of the dense 16-bit GEMV (`nq_dense_gemv_fwd`, the un-quantised `lm_head` of a decode step) with the
fp64 oracle on the exact stored values, through the C ABI (`ops.dense_gemv_forward`)."""
import pytest
import torch

from tests.util import TOL, exact_np

pytestmark = pytest.mark.gpu


def _case(T, N, V, dtype, seed, ldw=None, bias=False):
    g = torch.Generator().manual_seed(seed)
    ldw = ldw or N
    Wfull = (torch.randn((V, ldw), generator=g) * 0.05).to(dtype).cuda()
    W = Wfull[:, :N]
    x = torch.randn((T, N), generator=g).to(dtype).cuda()
    b = (torch.randn((V,), generator=g) * 0.5).to(dtype).cuda() if bias else None
    return x, W, b


def _check(x, W, b, y):
    from oracle import nanoquant_oracle as oc

    y64 = oc.dense_forward_fp64(exact_np(x), exact_np(W), exact_np(b) if b is not None else None)
    err = oc.rel_err(exact_np(y), y64)
    assert err <= TOL[x.dtype], err


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("T,N,V", [
    (1, 4096, 4000),      # V not a multiple of 16 rows
    (3, 2048, 1031),      # odd V, one batch per unit
    (8, 4096, 2048),
    (9, 1000, 777),       # N % 32 != 0: the last k block is half valid; two token blocks
    (16, 8192, 512),      # largest token count, four batches per unit
    (2, 8, 5),            # smallest legal shape
    (4, 5120, 16 * 700),  # more units than CTAs
])
def test_dense_gemv_matches_oracle(T, N, V, dtype):
    from nanoquant_b200 import ops

    x, W, b = _case(T, N, V, dtype, seed=T * 1000 + V)
    y = ops.dense_gemv_forward(x, W)
    assert y.shape == (T, V) and y.dtype == dtype
    _check(x, W, None, y)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dense_gemv_bias_row_stride_and_leading_dims(dtype):
    from nanoquant_b200 import ops

    x, W, b = _case(6, 1024, 1500, dtype, seed=5, ldw=1024 + 64, bias=True)
    assert not W.is_contiguous()
    y = ops.dense_gemv_forward(x.reshape(2, 3, 1024), W, b)
    assert y.shape == (2, 3, 1500)
    _check(x, W, b, y.reshape(6, 1500))


def test_dense_gemv_head_sized_against_fp32_matmul():
    """A 151936 x 4096 head (1.24 GB, the Qwen3-8B-shaped lm_head): compared with a chunked fp32 matmul of the same
    values on the GPU (the fp64 oracle of that size does not finish in seconds), and linear in x."""
    from nanoquant_b200 import ops

    V, N = 151936, 4096
    g = torch.Generator(device="cuda").manual_seed(11)
    W = (torch.randn((V, N), generator=g, device="cuda", dtype=torch.float32) * 0.02).to(torch.bfloat16)
    x = torch.randn((2, N), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    y = ops.dense_gemv_forward(x, W).float()
    ref = torch.cat([x.float() @ W[i:i + 16384].float().T for i in range(0, V, 16384)], dim=1)
    err = ((y - ref).abs().max() / ref.abs().max()).item()
    assert err <= TOL[torch.bfloat16], err
    # y(2 x) == 2 y(x) exactly: a power-of-two scale commutes with every rounding step
    y2 = ops.dense_gemv_forward((x * 2).contiguous(), W).float()
    assert torch.equal(y2, 2 * y)


def test_dense_gemv_errors():
    from nanoquant_b200 import _lib, ops

    L = _lib.lib()
    x, W, _ = _case(1, 64, 32, torch.float16, seed=1)
    y = torch.empty((1, 32), dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    call = lambda *a: L.nq_dense_gemv_fwd(*a)
    assert call(None, W.data_ptr(), None, y.data_ptr(), 1, 64, 32, 64, 32, 0, s) == _lib.NQ_ERR_NULL
    assert call(x.data_ptr(), W.data_ptr(), None, y.data_ptr(), 1, 60, 32, 64, 32, 0, s) == _lib.NQ_ERR_SHAPE
    assert call(x.data_ptr(), W.data_ptr(), None, y.data_ptr(), 1, 64, 32, 56, 32, 0, s) == _lib.NQ_ERR_SHAPE
    assert call(x.data_ptr(), W.data_ptr(), None, y.data_ptr(), 1, 64, 32, 64, 16, 0, s) == _lib.NQ_ERR_SHAPE
    assert call(x.data_ptr(), W.data_ptr(), None, y.data_ptr(), 1, 64, 32, 64, 32, 7, s) == _lib.NQ_ERR_DTYPE
    assert call(x.data_ptr() + 2, W.data_ptr(), None, y.data_ptr(), 1, 64, 32, 64, 32, 0, s) == _lib.NQ_ERR_ALIGN
    too_many = L.nq_dense_gemv_max_tokens() + 1
    assert call(x.data_ptr(), W.data_ptr(), None, y.data_ptr(), too_many, 64, 32, 64, 32, 0, s) == _lib.NQ_ERR_UNSUPPORTED
    with pytest.raises(RuntimeError):
        ops.dense_gemv_forward(x.float(), W)
    with pytest.raises(RuntimeError):
        ops.dense_gemv_forward(x[:, :32].contiguous(), W)
    torch.cuda.synchronize()


def test_dense_gemv_in_cuda_graph():
    from nanoquant_b200 import ops

    x, W, _ = _case(4, 2048, 3000, torch.bfloat16, seed=9)
    eager = ops.dense_gemv_forward(x, W)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ops.dense_gemv_forward(x, W)       # first call sets the kernel attribute outside capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = ops.dense_gemv_forward(x, W)
    y.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager)
