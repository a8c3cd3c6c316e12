"""The scratch-free GEMV entry point (``nq_gemv_fwd_static``) against ``nq_gemv_fwd``.

Some callers may not allocate device memory at the point where they run the layer (a fixed
memory plan, an allocator owned by the host application), so this entry point keeps its
intermediate in an array inside the library.  The test calls it through the C ABI twice in a
row - the second call meets the first call's leftovers in that array - and compares with the
regular entry point, which gets a fresh zeroed scratch buffer.  Collected last on purpose.
"""
import pytest
import torch

from oracle import nanoquant_oracle as oc
from tests.util import parity_excess, TOL, exact_np, half2_bits, make_layer

pytestmark = pytest.mark.gpu


def _run(entry, L, vt, ut, T, N, R, M, scratch=None):
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    y = torch.full((T, M), float("nan"), dtype=L["x"].dtype, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    dt = _lib.NQ_BF16 if L["x"].dtype == torch.bfloat16 else _lib.NQ_F16
    head = (L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
            L["s_post"].data_ptr(), y.data_ptr())
    if entry == "static":
        rc = Lb.nq_gemv_fwd_static(*head, T, N, R, M, dt, st)
    else:
        rc = Lb.nq_gemv_fwd(*head, scratch.data_ptr(), scratch.numel(), T, N, R, M, dt, st)
    _lib.check(rc, entry)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_static_scratch_entry_point_matches_regular_one(dtype):
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    Lb = _lib.lib()
    # 7 tokens: two launches on the shared array; rank 8192: the largest the array holds
    for (N, R, M, T) in ((1024, 288, 640, 3), (4096, 1600, 4096, 1), (1024, 288, 640, 7), (512, 8192, 64, 2)):
        L = make_layer(N, R, M, T, dtype, seed=R + T)
        vt = ku.pack_tiles(half2_bits(L["V"]), (R, N), "half2")
        ut = ku.pack_tiles(half2_bits(L["U"]), (M, R), "half2")
        scratch = torch.zeros(Lb.nq_gemv_scratch_bytes(T, N, R, M), dtype=torch.uint8, device="cuda")
        want = _run("regular", L, vt, ut, T, N, R, M, scratch)
        first = _run("static", L, vt, ut, T, N, R, M)
        second = _run("static", L, vt, ut, T, N, R, M)      # meets the first call's leftovers
        assert parity_excess(exact_np(want), L["y64"], dtype) <= 0
        # same kernel, exact integer accumulation: the results are identical, well inside the bar
        assert torch.equal(first, want) and torch.equal(second, want)
        # the array's status word is readable without its address: no wait gave up
        assert Lb.nq_scratch_status(None, torch.cuda.current_stream().cuda_stream) == 0


def test_static_scratch_entry_point_rejects_large_rank():
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    assert int(Lb.nq_gemv_static_max_rank()) == 8192
    big = int(Lb.nq_gemv_static_max_rank()) + 1
    z = torch.zeros(16, dtype=torch.uint8, device="cuda")
    rc = Lb.nq_gemv_fwd_static(z.data_ptr(), z.data_ptr(), z.data_ptr(), None, z.data_ptr(), z.data_ptr(),
                               z.data_ptr(), 1, 64, big, 64, _lib.NQ_F16, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.NQ_ERR_TOO_LARGE
    with pytest.raises(_lib.NanoQuantError, match="fixed maximum"):
        _lib.check(rc, "nq_gemv_fwd_static")
