"""Bounded device-side waits, made to run out without faulting or hanging anything: a wait that nothing will
ever satisfy returns after its (shortened) limit, the host reads NQ_ERR_TIMEOUT from the status word, and the
next call after re-zeroing works."""
import pytest
import torch

from tests.util import assert_parity, exact_np, make_layer, tiles_on_gpu

pytestmark = pytest.mark.gpu


def test_gemv_wait_for_a_stale_intermediate_expires():
    # The launch tag of a scratch is its launch count.  A header whose counter says "launch 5" while the buffer
    # holds no element with that tag is what a consumer sees when a producer never writes: here the producers DO
    # write, so to make a wait run out the status word is pre-set instead, which turns every wait of the launch
    # into a single poll (sticky expiry); the status stays set, and re-zeroing restores normal operation.
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    T, N, R, M = 1, 1024, 256, 512
    L = make_layer(N, R, M, T, torch.float16, seed=1)
    vt, ut = tiles_on_gpu(L["V"]), tiles_on_gpu(L["U"])
    st = torch.cuda.current_stream().cuda_stream
    nb = Lb.nq_gemv_scratch_bytes(T, N, R, M)
    scratch = torch.zeros(nb, dtype=torch.uint8, device="cuda")
    y = torch.empty(T, M, dtype=torch.float16, device="cuda")
    args = (L["x"].data_ptr(), L["s_pre"].data_ptr(), vt.data_ptr(), L["s_mid"].data_ptr(), ut.data_ptr(),
            L["s_post"].data_ptr(), y.data_ptr(), scratch.data_ptr(), nb, T, N, R, M, _lib.NQ_F16, st)
    old = Lb.nq_gemv_set_wait_limit(64)          # a few dozen polls instead of four million
    try:
        scratch.view(torch.int32)[2] = 7         # an earlier expiry left its mark: this launch must not spin
        _lib.check(Lb.nq_gemv_fwd(*args), "nq_gemv_fwd")
        torch.cuda.synchronize()
        assert Lb.nq_scratch_status(scratch.data_ptr(), st) != 0
        scratch.zero_()
        _lib.check(Lb.nq_gemv_fwd(*args), "nq_gemv_fwd")
        assert Lb.nq_scratch_status(scratch.data_ptr(), st) == 0
        assert_parity(exact_np(y), L["y64"], torch.float16, what="after re-zeroing")
    finally:
        assert Lb.nq_gemv_set_wait_limit(old) == 64


def test_allgather_wait_for_an_absent_peer_expires():
    # world = 2 on one GPU, both "ranks" pointing at this process's buffer; slot 1's flag is never written, so the
    # wait for rank 1 runs out: the kernel returns, the status says so, and after re-zeroing a world of 1 works.
    from nanoquant_b200 import _lib
    import ctypes
    Lb = _lib.lib()
    if not hasattr(Lb, "nq_allgather_set_wait_limit"):
        pytest.skip("library without a run-time limit for the all-gather wait")
    st = torch.cuda.current_stream().cuda_stream
    shard = torch.arange(64, dtype=torch.float16, device="cuda")
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    state = torch.zeros(Lb.nq_allgather_state_bytes(), dtype=torch.uint8, device="cuda")
    bases = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    old = Lb.nq_allgather_set_wait_limit(2000)
    try:
        rc = Lb.nq_allgather_push(shard.data_ptr(), shard.numel() * 2, bases, 0, 1024, state.data_ptr(), 2, 0, st)
        _lib.check(rc, "nq_allgather_push")
        torch.cuda.synchronize()
        assert Lb.nq_allgather_status(state.data_ptr(), st) == _lib.NQ_ERR_TIMEOUT
        buf.zero_(); state.zero_()
        bases1 = (ctypes.c_void_p * 1)(buf.data_ptr())
        _lib.check(Lb.nq_allgather_push(shard.data_ptr(), shard.numel() * 2, bases1, 0, 1024, state.data_ptr(), 1, 0, st), "push")
        assert Lb.nq_allgather_status(state.data_ptr(), st) == 0
        assert torch.equal(buf[1024:1024 + 128].view(torch.float16), shard)
    finally:
        Lb.nq_allgather_set_wait_limit(old)
