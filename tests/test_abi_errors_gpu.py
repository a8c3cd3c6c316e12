"""Error behaviour of the C ABI: every misuse returns a negative status, nothing is launched, nothing faults."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    from nanoquant_b200 import _lib
    L = _lib.lib()
    z = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    return _lib, L, z, torch.cuda.current_stream().cuda_stream


def test_gemv_argument_checks(env):
    _lib, L, z, st = env
    p = z.data_ptr()
    y, sc = p + 8192, p + 16384          # separate regions for the output and the scratch
    n = L.nq_gemv_scratch_bytes(1, 64, 32, 32)
    call = lambda **kw: L.nq_gemv_fwd(kw.get("x", p), p, p, None, p, p, y, kw.get("scratch", sc), kw.get("nbytes", n),
                                      kw.get("T", 1), kw.get("N", 64), kw.get("R", 32), kw.get("M", 32),
                                      kw.get("dtype", _lib.NQ_F16), st)
    assert call() == _lib.NQ_OK
    assert call(x=None) == _lib.NQ_ERR_NULL
    assert call(T=0) == _lib.NQ_ERR_SHAPE
    assert call(N=-5) == _lib.NQ_ERR_SHAPE
    assert call(dtype=7) == _lib.NQ_ERR_DTYPE
    assert call(nbytes=n - 1) == _lib.NQ_ERR_SCRATCH
    assert call(scratch=sc + 4) == _lib.NQ_ERR_ALIGN
    assert call(N=40000) == _lib.NQ_ERR_UNSUPPORTED         # beyond the 32768-column limit of the fixed-point sums
    assert L.nq_gemv_scratch_bytes(0, 64, 32, 32) == 0
    torch.cuda.synchronize()
    assert L.nq_scratch_status(sc, st) == _lib.NQ_OK


def test_group_limits(env):
    _lib, L, z, st = env
    p = z.data_ptr()
    d = (_lib.LinearDesc * 5)(*[_lib.LinearDesc(p, p, p, None, p, p, p, 64, 32, 32, 64, 32) for _ in range(5)])
    assert L.nq_gemv_group_fwd(d, 5, 1, _lib.NQ_F16, p, z.numel(), st) == _lib.NQ_ERR_UNSUPPORTED   # at most 4 linears
    assert L.nq_gemv_group_fwd(d, 0, 1, _lib.NQ_F16, p, z.numel(), st) == _lib.NQ_ERR_UNSUPPORTED
    bad = (_lib.LinearDesc * 1)(_lib.LinearDesc(p, p, p, None, p, p, p, 64, 32, 32, 32, 32))        # ldx < N
    assert L.nq_gemv_group_fwd(bad, 1, 1, _lib.NQ_F16, p, z.numel(), st) == _lib.NQ_ERR_SHAPE


def test_gemm_argument_checks(env):
    _lib, L, z, st = env
    p = z.data_ptr()
    y, sc = p + 8192, p + 16384
    n = L.nq_gemm_scratch_bytes(16, 64, 32, 32)
    assert L.nq_gemm_fwd(p, p, p, None, p, p, y, sc, n, 16, 64, 32, 32, _lib.NQ_BF16, st) == _lib.NQ_OK
    assert L.nq_gemm_fwd(p, p, p, None, p, p, y, sc, n - 1, 16, 64, 32, 32, _lib.NQ_BF16, st) == _lib.NQ_ERR_SCRATCH
    assert L.nq_gemm_fwd(p, p, p, None, p, p, y, sc, n, 16, 60, 32, 32, _lib.NQ_BF16, st) == _lib.NQ_ERR_SHAPE  # N % 8
    assert L.nq_gemm_fwd(p + 2, p, p, None, p, p, y, sc, n, 16, 64, 32, 32, _lib.NQ_BF16, st) == _lib.NQ_ERR_ALIGN
    assert L.nq_onebit_gemm_fwd(p, p, None, None, p, None, 16, 64, 32, _lib.NQ_F16, st) == _lib.NQ_ERR_NULL
    torch.cuda.synchronize()


def test_pack_argument_checks(env):
    _lib, L, z, st = env
    p = z.data_ptr()
    assert L.nq_pack_rows(p, p, 4, 64, 9, st) == _lib.NQ_ERR_DTYPE
    assert L.nq_pack_rows(None, p, 4, 64, 0, st) == _lib.NQ_ERR_NULL
    assert L.nq_pack_rows(None, None, 0, 64, 0, st) == _lib.NQ_OK            # empty matrix: nothing to do
    assert L.nq_pack_marlin(p, p, 65, 16, st) == _lib.NQ_ERR_SHAPE
    assert L.nq_permute_scale16(p, p, 32, 1, 0, st) == _lib.NQ_ERR_UNSUPPORTED   # in place
    assert L.nq_permute_scale16(p, p + 1024, 30, 1, 0, st) == _lib.NQ_ERR_SHAPE
    assert L.nq_rows_to_tiles(p, p + 4, 16, 256, 0, st) == _lib.NQ_ERR_ALIGN
    assert L.nq_tiles_bytes(16, 256) == 512 and L.nq_tiles_bytes(17, 257) == 4 * 512 and L.nq_tiles_bytes(0, 5) == 0
    for code in range(0, -10, -1):
        assert L.nq_strerror(code)
    torch.cuda.synchronize()


def test_zero_tokens_through_the_operators():
    import binary_kernels  # noqa: F401
    from tests.util import half2_bits, make_layer
    L = make_layer(256, 64, 128, 1, torch.float16, seed=1)
    y = torch.ops.binary_kernels.nanoquant_dyn_forward(L["x"][:0], L["s_pre"], half2_bits(L["V"]), L["s_mid"],
                                                       half2_bits(L["U"]), L["s_post"], num_acc_stage1=1, num_acc_stage2=1)
    assert y.shape == (0, 128)


def test_peer_all_gather_on_one_gpu(env):
    """nq_allgather_push with a world of one (the rank's own buffer is the only "peer"): the shard lands in
    slot 0 of the region, repeated launches advance the epoch, arguments are checked."""
    import ctypes
    _lib, L, z, st = env
    dev = z.device
    flags = L.nq_allgather_flags_bytes(1)
    assert flags == 256 and L.nq_allgather_flags_bytes(9) == 0
    arena = torch.zeros(flags + 3 * 4096, dtype=torch.uint8, device=dev)
    state = torch.zeros(L.nq_allgather_state_bytes(), dtype=torch.uint8, device=dev)
    bases = (ctypes.c_void_p * 1)(arena.data_ptr())
    for rep, nbytes in enumerate((16, 4096, 1040)):
        shard = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev)
        off = flags + rep * 4096
        assert L.nq_allgather_push(shard.data_ptr(), nbytes, bases, 0, off, state.data_ptr(), 1, 0, st) == _lib.NQ_OK
        assert L.nq_allgather_status(state.data_ptr(), st) == _lib.NQ_OK
        assert torch.equal(arena[off:off + nbytes], shard)
        assert int(arena[:4].view(torch.int32)[0]) == rep + 1           # this rank's flag word holds the epoch
    shard = torch.zeros(64, dtype=torch.uint8, device=dev)
    args = lambda **kw: dict(dict(shard=shard.data_ptr(), n=64, bases=bases, fo=0, ro=flags, state=state.data_ptr(), world=1, rank=0), **kw)
    call = lambda a: L.nq_allgather_push(a["shard"], a["n"], a["bases"], a["fo"], a["ro"], a["state"], a["world"], a["rank"], st)
    assert call(args(n=40)) == _lib.NQ_ERR_ALIGN          # not a multiple of 16 bytes
    assert call(args(ro=flags + 8)) == _lib.NQ_ERR_ALIGN
    assert call(args(world=9)) == _lib.NQ_ERR_SHAPE
    assert call(args(rank=1)) == _lib.NQ_ERR_SHAPE
    assert call(args(state=None)) == _lib.NQ_ERR_NULL
    torch.cuda.synchronize()
