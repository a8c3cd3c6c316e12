"""The numpy oracle against fixtures produced by running the reference
(``tests/golden/make_golden.py``).  CPU only."""
import os

import numpy as np
import pytest

from oracle import nanoquant_oracle as oc


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


@pytest.mark.parametrize("method", ["lsb_first", "half2"])
def test_pack_rows_bit_exact(golden_dir, method):
    g = load(golden_dir, "pack_rows.npz")
    for name in "abcde":
        w = g[f"{name}_w"]
        want = g[f"{name}_{method}"]
        got = oc.pack_rows(w, method)
        assert got.dtype == np.int32 and got.shape == want.shape
        assert np.array_equal(got, want)
        assert np.array_equal(oc.unpack_rows(want, w.shape, method), w)


@pytest.mark.parametrize("method", ["lsb_first", "half2"])
def test_pack_onehot_known_answers(golden_dir, method):
    g = load(golden_dir, "pack_onehot.npz")
    for c, want in zip(g["cols"], g[method]):
        w = np.ones((1, 64), np.int8)
        w[0, c] = -1
        assert np.array_equal(oc.pack_rows(w, method)[0], want)
    # the literal known answers of the two layouts
    w = np.ones((1, 32), np.int8); w[0, 0] = -1
    assert oc.pack_rows(w, "lsb_first").view(np.uint32)[0, 0] == 0x1
    assert oc.pack_rows(w, "half2").view(np.uint32)[0, 0] == 0x8000
    w = np.ones((1, 32), np.int8); w[0, 31] = -1
    assert oc.pack_rows(w, "lsb_first").view(np.uint32)[0, 0] == 0x80000000
    assert oc.pack_rows(w, "half2").view(np.uint32)[0, 0] == 0x10000


def test_pack_rows_errors():
    with pytest.raises(TypeError):
        oc.pack_rows(np.ones((2, 2), np.int32))
    with pytest.raises(ValueError):
        oc.pack_rows(np.ones((2, 2), np.int8), "msb")
    with pytest.raises(ValueError):
        oc.unpack_rows(np.zeros((2, 2), np.int32), (2, 32))


def test_pack_marlin_bit_exact(golden_dir):
    g = load(golden_dir, "pack_marlin.npz")
    for name in "abc":
        B, si, so, ws = oc.pack_marlin(g[f"{name}_w"], g[f"{name}_s_in"], g[f"{name}_s_out"])
        assert np.array_equal(B, g[f"{name}_B"])
        assert np.array_equal(si, g[f"{name}_s_in_p"])
        assert np.array_equal(so, g[f"{name}_s_out_p"])
        assert ws == int(g[f"{name}_ws"])
    for (o, i), want in zip(g["hot_idx"], g["hot_B"]):
        w = np.ones((128, 32), np.int8)
        w[o, i] = -1
        assert np.array_equal(oc.pack_marlin_bits(w), want)


def test_pack_marlin_fused_bit_exact(golden_dir):
    g = load(golden_dir, "pack_marlin_fused.npz")
    Vb, Ub, s1, s2, s3, ws = oc.pack_marlin_fused(g["V_sign"], g["U_sign"], g["sg"], g["sl"], g["sh"])
    for got, key in ((Vb, "Vb"), (Ub, "Ub"), (s1, "s1"), (s2, "s2"), (s3, "s3"), (ws, "ws")):
        assert got.shape == g[key].shape, key
        assert np.array_equal(got, g[key]), key


def test_forward_fp64_matches_reference_module(golden_dir):
    g = load(golden_dir, "forward_fp64.npz")
    for name in "abc":
        s_mid = g[f"{name}_s_mid"] if f"{name}_s_mid" in g else None
        y = oc.forward_fp64(g[f"{name}_x"], g[f"{name}_V"], g[f"{name}_U"],
                            g[f"{name}_s_pre"], s_mid, g[f"{name}_s_post"])
        assert np.allclose(y, g[f"{name}_y"], rtol=1e-12, atol=0)
        # checkpoint layout of the module's own state_dict
        V, U = g[f"{name}_V"], g[f"{name}_U"]
        assert np.array_equal(oc.pack_rows(V, "lsb_first"), g[f"{name}_V_packed"])
        assert np.array_equal(oc.pack_rows(U, "lsb_first"), g[f"{name}_U_packed"])
        assert tuple(g[f"{name}_V_shape"]) == V.shape and tuple(g[f"{name}_U_shape"]) == U.shape


def test_forward_bf16_reference_within_bf16_error(golden_dir):
    g = load(golden_dir, "forward_bf16.npz")
    y = oc.forward_fp64(g["x"], g["V"], g["U"], g["s_pre"], g["s_mid"], g["s_post"])
    # the reference module computes in bf16: three roundings of 2^-9 each plus accumulation
    assert oc.rel_err(g["y"], y) < 2e-2


def test_rank_formula(golden_dir):
    for a, b, bits, ns, want in load(golden_dir, "ranks.npz")["table"]:
        assert oc.rank_for_bits(int(a), int(b), float(bits), int(ns)) == int(want)
    assert oc.rank_for_bits(4096, 4096, 0.8) == 1600
    assert oc.rank_for_bits(4096, 12288, 0.8) == 2432
    assert oc.rank_for_bits(4096, 1024, 0.8) == 608


def test_forward_from_packed_roundtrip():
    d = oc.synth_linear(96, 64, 40, 3, seed=1)
    y = oc.forward_fp64(d["x"], d["V"], d["U"], d["s_pre"], d["s_mid"], d["s_post"])
    for method in ("lsb_first", "half2"):
        y2 = oc.forward_from_packed(d["x"], oc.pack_rows(d["V"], method), oc.pack_rows(d["U"], method),
                                    d["s_pre"], d["s_mid"], d["s_post"], 96, 64, 40, method)
        assert np.array_equal(y, y2)


def test_dense_forward_is_torch_linear():
    """The un-quantised head is an ``nn.Linear`` in the reference (``utils/load_utils.py:322``): the oracle's dense
    forward must be ``torch.nn.functional.linear`` evaluated in float64 on the same bf16 values."""
    import torch

    g = torch.Generator().manual_seed(7)
    x = torch.randn((5, 192), generator=g).to(torch.bfloat16)
    W = (torch.randn((77, 192), generator=g) * 0.05).to(torch.bfloat16)
    b = torch.randn((77,), generator=g).to(torch.bfloat16)
    to64 = lambda t: t.float().numpy().astype(np.float64)
    for bias in (None, b):
        want = torch.nn.functional.linear(x.double(), W.double(), None if bias is None else bias.double()).numpy()
        got = oc.dense_forward_fp64(to64(x), to64(W), None if bias is None else to64(bias))
        assert np.allclose(got, want, rtol=1e-13, atol=1e-15)
        # and the bf16 module output agrees with it within bf16 rounding
        y16 = torch.nn.functional.linear(x, W, bias).float().numpy()
        assert oc.rel_err(y16, got) < 2.0 ** -7
