"""Pack / layout kernels through the C ABI against the numpy oracle and the
golden fixtures produced by the reference.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import nanoquant_oracle as oc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ku():
    from nanoquant_b200.kernel import utils
    return utils


def signs(shape, seed):
    g = np.random.default_rng(seed)
    return (g.integers(0, 2, size=shape, dtype=np.int8) * 2 - 1).astype(np.int8)


SHAPES = [(1, 1), (5, 32), (7, 70), (16, 257), (3, 96), (64, 4096), (33, 1000), (1536, 4096), (129, 31)]


@pytest.mark.parametrize("method", ["lsb_first", "half2"])
@pytest.mark.parametrize("shape", SHAPES)
def test_pack_unpack_rows_vs_oracle(ku, method, shape):
    w = signs(shape, seed=shape[0] * 131 + shape[1])
    wt = torch.from_numpy(w).cuda()
    got = ku.pack_binary_gemv(wt, method=method)
    want = oc.pack_rows(w, method)
    assert got.dtype == torch.int32 and tuple(got.shape) == want.shape
    assert np.array_equal(got.cpu().numpy(), want)
    back = ku.unpack_binary_gemv(got, shape, method=method)
    assert back.dtype == torch.int8 and np.array_equal(back.cpu().numpy(), w)


@pytest.mark.parametrize("method", ["lsb_first", "half2"])
def test_pack_rows_golden(ku, golden_dir, method):
    g = np.load(os.path.join(golden_dir, "pack_rows.npz"))
    for name in "abcde":
        w = torch.from_numpy(g[f"{name}_w"])
        got = ku.pack_binary_gemv(w, method=method)            # CPU tensor: staged through the GPU
        assert got.device.type == "cpu"
        assert np.array_equal(got.numpy(), g[f"{name}_{method}"])
    g = np.load(os.path.join(golden_dir, "pack_onehot.npz"))
    for c, want in zip(g["cols"], g[method]):
        w = torch.ones(1, 64, dtype=torch.int8, device="cuda")
        w[0, int(c)] = -1
        assert np.array_equal(ku.pack_binary_gemv(w, method=method).cpu().numpy()[0], want)


def test_pack_rows_unaligned_view(ku):
    # a storage offset that breaks 16-byte alignment takes the scalar path
    w = signs((9, 64), 5)
    buf = torch.zeros(9 * 64 + 3, dtype=torch.int8, device="cuda")
    buf[3:] = torch.from_numpy(w).reshape(-1).cuda()
    view = buf[3:].view(9, 64)
    assert np.array_equal(ku.pack_binary_gemv(view).cpu().numpy(), oc.pack_rows(w))


def test_pack_rows_errors(ku):
    with pytest.raises(TypeError):
        ku.pack_binary_gemv(torch.ones(2, 2, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        ku.pack_binary_gemv(torch.ones(2, 2, dtype=torch.int8, device="cuda"), method="msb")
    with pytest.raises(ValueError):
        ku.unpack_binary_gemv(torch.zeros(2, 2, dtype=torch.int32, device="cuda"), (2, 32))
    with pytest.raises(ValueError):
        ku.unpack_binary_gemv(torch.zeros(4, dtype=torch.int32, device="cuda"), (2, 64))


def test_empty_inputs(ku):
    out = ku.pack_binary_gemv(torch.empty(0, 64, dtype=torch.int8, device="cuda"))
    assert tuple(out.shape) == (0, 2)
    out = ku.unpack_binary_gemv(torch.empty(0, 2, dtype=torch.int32, device="cuda"), (0, 64))
    assert tuple(out.shape) == (0, 64)


def test_reorder_words(ku):
    w = signs((40, 320), 9)
    lsb = torch.from_numpy(oc.pack_rows(w, "lsb_first")).cuda()
    h2 = torch.from_numpy(oc.pack_rows(w, "half2")).cuda()
    assert torch.equal(ku.reorder_packed(lsb, "lsb_first", "half2"), h2)
    assert torch.equal(ku.reorder_packed(h2, "half2", "lsb_first"), lsb)
    assert torch.equal(ku.reorder_packed(h2, "half2", "half2"), h2)
    odd = lsb.reshape(-1)[:397].contiguous()          # a word count that is not a multiple of four: scalar kernel
    assert torch.equal(ku.reorder_packed(odd[None], "lsb_first", "half2")[0], h2.reshape(-1)[:397])


def test_pack_marlin_golden_and_oracle(ku, golden_dir):
    g = np.load(os.path.join(golden_dir, "pack_marlin.npz"))
    for name in "abc":
        w = torch.from_numpy(g[f"{name}_w"]).cuda()
        B, si, so, ws = ku.pack_binary_marlin(w, torch.from_numpy(g[f"{name}_s_in"]).cuda(),
                                              torch.from_numpy(g[f"{name}_s_out"]).cuda())
        assert np.array_equal(B.cpu().numpy(), g[f"{name}_B"])
        assert np.array_equal(si.cpu().numpy(), g[f"{name}_s_in_p"])
        assert np.array_equal(so.cpu().numpy(), g[f"{name}_s_out_p"])
        assert ws == int(g[f"{name}_ws"])
    for (o, i), want in zip(g["hot_idx"], g["hot_B"]):
        w = torch.ones(128, 32, dtype=torch.int8, device="cuda")
        w[int(o), int(i)] = -1
        B, _, _, _ = ku.pack_binary_marlin(w, torch.ones(32, dtype=torch.float16, device="cuda"),
                                           torch.ones(128, dtype=torch.float16, device="cuda"))
        assert np.array_equal(B.cpu().numpy(), want)
    w = signs((1536, 4096), 11)
    B, _, _, _ = ku.pack_binary_marlin(torch.from_numpy(w).cuda(),
                                       torch.ones(4096, dtype=torch.float16, device="cuda"),
                                       torch.ones(1536, dtype=torch.float16, device="cuda"))
    assert np.array_equal(B.cpu().numpy(), oc.pack_marlin_bits(w))


def test_pack_marlin_partial_blocks_and_unaligned_base(ku):
    # in_f not a multiple of the 128 columns a CTA stages (partial last block), and a base pointer that is not
    # 16-byte aligned (the byte-wise kernel takes over): both bit-exact with the oracle
    from nanoquant_b200 import _lib
    Lb = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    for (o, i) in [(128, 208), (192, 16), (64, 400)]:
        w = signs((o, i), o + i)
        want = oc.pack_marlin_bits(w)
        for offset in (0, 1):
            buf = torch.zeros(o * i + 16, dtype=torch.int8, device="cuda")
            buf[offset:offset + o * i] = torch.from_numpy(w).reshape(-1).cuda()
            B = torch.empty(i // 16, o // 2, dtype=torch.int32, device="cuda")
            _lib.check(Lb.nq_pack_marlin(buf.data_ptr() + offset, B.data_ptr(), o, i, st), "nq_pack_marlin")
            assert np.array_equal(B.cpu().numpy(), want), (o, i, offset)


def test_pack_marlin_fused_golden(ku, golden_dir):
    g = np.load(os.path.join(golden_dir, "pack_marlin_fused.npz"))
    t = lambda k: torch.from_numpy(g[k]).cuda()
    out = ku.pack_binary_marlin_fused(t("V_sign"), t("U_sign"), t("sg"), t("sl"), t("sh"))
    for got, key in zip(out, ("Vb", "Ub", "s1", "s2", "s3", "ws")):
        assert tuple(got.shape) == g[key].shape, key
        assert np.array_equal(got.cpu().numpy(), g[key]), key


def test_marlin_to_rows_roundtrip(ku):
    from nanoquant_b200 import _lib
    w = signs((192, 160), 13)
    B = torch.from_numpy(oc.pack_marlin_bits(w)).cuda()
    for method in ("lsb_first", "half2"):
        out = torch.empty(192, 5, dtype=torch.int32, device="cuda")
        _lib.check(_lib.lib().nq_marlin_to_rows(B.data_ptr(), out.data_ptr(), 192, 160, _lib.ORDER_ID[method],
                                                torch.cuda.current_stream().cuda_stream), "nq_marlin_to_rows")
        assert np.array_equal(out.cpu().numpy(), oc.pack_rows(w, method))


def tiles_reference(w):
    """The tile layout written out from its definition (slow, small cases)."""
    rows, cols = w.shape
    rgs, chunks = (rows + 15) // 16, (cols + 255) // 256
    out = np.zeros((rgs, chunks, 32, 4), dtype=np.uint32)
    for r in range(rows):
        for k in range(cols):
            if w[r, k] < 0:
                rg, rr = divmod(r, 16)
                g, half_row = rr % 8, rr // 8
                c, kk = divmod(k, 256)
                j, k32 = divmod(kk, 32)
                h, k16 = divmod(k32, 16)
                q, b = divmod(k16, 4)
                out[rg, c, 4 * g + q, 2 * h + half_row] |= np.uint32(1) << np.uint32(8 * b + j)
    return out.reshape(rgs, chunks, 128).view(np.int32)


@pytest.mark.parametrize("shape", [(16, 256), (40, 300), (33, 1000), (96, 512), (7, 31)])
def test_tiles_layout(ku, shape):
    w = signs(shape, shape[0] + shape[1])
    want = tiles_reference(w)
    for method in ("lsb_first", "half2"):
        packed = torch.from_numpy(oc.pack_rows(w, method)).cuda()
        tiles = ku.pack_tiles(packed, shape, method)
        assert np.array_equal(tiles.cpu().numpy(), want)
        assert torch.equal(ku.unpack_tiles(tiles, shape, method), packed)


def test_tiles_roundtrip_large(ku):
    w = signs((4096, 1536), 3)
    packed = torch.from_numpy(oc.pack_rows(w, "half2")).cuda()
    tiles = ku.pack_tiles(packed, (4096, 1536), "half2")
    assert tuple(tiles.shape) == (256, 6, 128)
    assert torch.equal(ku.unpack_tiles(tiles, (4096, 1536), "half2"), packed)


def test_scale_permutation_inverse(ku):
    s = torch.randn(96, device="cuda").to(torch.bfloat16)
    for kind in (0, 1):
        p = ku._permute_scale(s, kind)
        assert torch.equal(ku._permute_scale(p, kind, inverse=True), s)
    ref = oc.marlin_perm_scale_out(s.float().cpu().numpy())
    assert np.array_equal(ku._permute_scale(s, 1).float().cpu().numpy(), ref)
