"""Model-level pieces around the quantised linear: the compressed-checkpoint loader (save -> load -> forward
round trip without dense factors), launch groups, a toy decoder layer whose whole step is replayed from a CUDA
graph, and the operators under ``torch.compile`` as the reference's decode benchmark runs them
(``src/nanoquant/kernel/test_decode.py:396-402``)."""
import io

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import nanoquant_oracle as oc
from tests.util import assert_parity, exact_np

pytestmark = pytest.mark.gpu

DT = torch.bfloat16


def fill(m, d):
    with torch.no_grad():
        m.V.copy_(torch.from_numpy(d["V"]).float())
        m.U.copy_(torch.from_numpy(d["U"]).float())
        m.scale_pre.copy_(torch.from_numpy(d["s_pre"]).float()[None])
        if hasattr(m, "scale_mid") and m.scale_mid is not None:
            m.scale_mid.copy_(torch.from_numpy(d["s_mid"]).float()[None])
        m.scale_post.copy_(torch.from_numpy(d["s_post"]).float()[None])


def bf(a):
    """float64 image of a numpy array rounded to bf16, as the module keeps its scales."""
    return exact_np(torch.from_numpy(np.asarray(a, np.float32)).to(DT))


class ToyLayer(nn.Module):
    """RMSNorm -> q/k/v, o, RMSNorm -> gate/up -> SiLU*up -> down with residuals: the linears of a decoder layer
    (attention itself replaced by the identity on v, which keeps the data flow and needs no cache)."""

    def __init__(self, H=256, I=512, KV=128):
        super().__init__()
        self.H, self.I, self.KV = H, I, KV
        mk = lambda n, m: nn.Linear(n, m, bias=False)
        self.q, self.k, self.v, self.o = mk(H, H), mk(H, KV), mk(H, KV), mk(KV, H)
        self.gate, self.up, self.down = mk(H, I), mk(H, I), mk(I, H)
        self.lm_head = mk(H, 1000)
        self.norm1 = nn.Parameter(torch.ones(H))
        self.norm2 = nn.Parameter(torch.ones(H))

    @staticmethod
    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(x.dtype)

    def forward(self, x):          # module by module, as the reference's model forward does
        h = self.rms(x, self.norm1)
        a = self.o(self.v(h) + 0 * self.q(h)[..., :self.KV] + 0 * self.k(h))
        x = x + a
        h = self.rms(x, self.norm2)
        x = x + self.down(torch.nn.functional.silu(self.gate(h)) * self.up(h))
        return x


QUANT = ("q", "k", "v", "o", "gate", "up", "down")


def quantised_toy(seed=0, with_mid=True):
    from nanoquant_b200.modules.linear import NanoQuantLinear
    torch.manual_seed(seed)
    m = ToyLayer()
    data = {}
    for i, name in enumerate(QUANT):
        lin = getattr(m, name)
        N, M = lin.in_features, lin.out_features
        R = 64 if name in ("k", "v") else 96
        d = oc.synth_linear(N, R, M, 1, seed=seed + i)
        d["s_post"] = (d["s_post"].astype(np.float32) * 30).astype(d["s_post"].dtype)   # outputs of order one
        q = NanoQuantLinear(N, M, R, has_scale_mid=with_mid)
        fill(q, d)
        setattr(m, name, q)
        data[name] = d
    with torch.no_grad():
        m.norm1.copy_(torch.rand(m.H) + 0.5)
        m.norm2.copy_(torch.rand(m.H) + 0.5)
    return m, data


def test_checkpoint_round_trip_without_dense_factors(tmp_path):
    from nanoquant_b200.modules.linear import NanoQuantLinear
    from nanoquant_b200.utils.load_utils import get_compressed_state_dict, load_compressed_checkpoint
    src, data = quantised_toy(seed=3)
    sd = get_compressed_state_dict(src)
    assert "q.V_packed" in sd and "q.V" not in sd and "lm_head.weight" in sd and "norm1" in sd
    assert sd["down.U_packed"].dtype == torch.int32 and tuple(sd["down.U_shape"].tolist()) == (256, 96)
    path = tmp_path / "ckpt.pt"
    torch.save(sd, path)
    for kernel_type, T in (("gemv", 2), ("gemm", 70)):
        dst = ToyLayer()                                   # plain nn.Linear everywhere, as AutoModel.from_config gives
        load_compressed_checkpoint(dst, str(path), dtype=DT, device="cuda", kernel_type=kernel_type)
        assert isinstance(dst.q, NanoQuantLinear) and type(dst.lm_head) is nn.Linear
        assert not hasattr(dst.q, "V") and dst.q.V_int8.dim() == 3 and dst.q.V_int8.is_cuda
        assert torch.equal(dst.lm_head.weight.cpu(), src.lm_head.weight) and dst.norm1.is_cuda
        x = torch.randn(T, 256, generator=torch.Generator().manual_seed(T)).to(DT).cuda()
        for name in ("q", "down"):
            d = data[name]
            xin = x if name == "q" else torch.randn(T, 512, generator=torch.Generator().manual_seed(9)).to(DT).cuda()
            y = getattr(dst, name)(xin)
            y64 = oc.forward_fp64(exact_np(xin), d["V"], d["U"], bf(d["s_pre"]), bf(d["s_mid"]), bf(d["s_post"]))
            assert_parity(exact_np(y), y64, DT, what=f"{kernel_type} {name}")


def test_launch_group_equals_separate_modules():
    from nanoquant_b200.modules.group import LinearGroup
    m, _ = quantised_toy(seed=5, with_mid=False)      # no scale_mid: ranks 64 / 96 must come from the modules
    m = m.cuda()
    for name in QUANT:
        getattr(m, name)._prepare_kernel("gemv", DT)
    for T in (1, 4, 9):                                 # 9 tokens: the group GEMM
        x = torch.randn(T, m.H, generator=torch.Generator().manual_seed(T)).to(DT).cuda()
        q, k, v = LinearGroup([m.q, m.k, m.v])(x)
        assert torch.equal(q, m.q(x)) if T <= 4 else oc.rel_err(exact_np(q), exact_np(m.q(x))) < 2 ** -7
        assert torch.equal(k, m.k(x)) if T <= 4 else oc.rel_err(exact_np(k), exact_np(m.k(x))) < 2 ** -7
        assert torch.equal(v, m.v(x)) if T <= 4 else oc.rel_err(exact_np(v), exact_np(m.v(x))) < 2 ** -7
        # residual in the epilogue of a one-linear group
        (o,) = LinearGroup([m.o])(v, residuals=[x])
        ref = (m.o(v).float() + x.float())
        assert oc.rel_err(exact_np(o), ref.double().cpu().numpy()) < 2 ** -7
    x3 = torch.randn(2, 3, m.H).to(DT).cuda()           # [batch, seq, hidden] input keeps its leading dimensions
    g, u = LinearGroup([m.gate, m.up])(x3)
    assert g.shape == (2, 3, m.I) and torch.equal(g, m.gate(x3))


def grouped_step(m, groups, x):
    """The toy layer with folded norm weights, launch groups and residuals in the epilogues: 4 launches."""
    xf = x.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype)     # norm weight folded into scale_pre
    q, k, v = groups["qkv"](h)
    (x1,) = groups["o"](v, residuals=[x])                                           # x + o(v)
    xf = x1.float()
    h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).to(x.dtype)
    g, u = groups["gu"](h)
    (x2,) = groups["down"](torch.nn.functional.silu(g) * u, residuals=[x1])
    return x2


def test_toy_decoder_layer_grouped_graph_equals_eager_modules():
    from nanoquant_b200.modules.group import LinearGroup
    from nanoquant_b200 import ops
    m, _ = quantised_toy(seed=7)
    m = m.cuda()
    ref, _ = quantised_toy(seed=7)
    ref = ref.cuda()
    for name in QUANT:
        getattr(ref, name)._prepare_kernel("gemv", DT)
    # fold the RMSNorm weights into the input scales of the linears they feed, then prepare
    for name in ("q", "k", "v"):
        getattr(m, name).fold_input_scale(m.norm1.data)
    for name in ("gate", "up"):
        getattr(m, name).fold_input_scale(m.norm2.data)
    for name in QUANT:
        getattr(m, name)._prepare_kernel("gemv", DT)
    groups = {"qkv": LinearGroup([m.q, m.k, m.v]), "o": LinearGroup([m.o]), "gu": LinearGroup([m.gate, m.up]),
              "down": LinearGroup([m.down])}
    x = torch.randn(1, m.H, generator=torch.Generator().manual_seed(1)).to(DT).cuda()
    with torch.no_grad():
        y_ref = ref(x)
        y_eager = grouped_step(m, groups, x)
        head = ops.dense_gemv_forward(y_eager, m.lm_head.weight.to(DT))
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            grouped_step(m, groups, x)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                y_graph = grouped_step(m, groups, x)
                head_graph = ops.dense_gemv_forward(y_graph, m.lm_head.weight.to(DT))
            graph.replay()
            graph.replay()
        torch.cuda.synchronize()
    assert torch.equal(y_graph, y_eager) and torch.equal(head_graph, head)
    # folding the norm weight changes where one rounding happens, nothing else
    assert oc.rel_err(exact_np(y_eager), exact_np(y_ref)) < 2 ** -6


def test_operators_under_torch_compile():
    m, data = quantised_toy(seed=11)
    m = m.cuda()
    for name in QUANT:
        getattr(m, name)._prepare_kernel("gemv", DT)
    x = torch.randn(1, m.H, generator=torch.Generator().manual_seed(2)).to(DT).cuda()
    with torch.no_grad():
        y_eager = m(x)
        # the reference's call (test_decode.py:396-402): inductor with CUDA graphs; the fake implementations of the
        # operators make the module traceable as one graph, and nothing allocates inside the replayed region
        fn = torch.compile(m, mode="reduce-overhead", fullgraph=True)
        outs = [fn(x).clone() for _ in range(4)]        # warm-up, capture, replays
        fn2 = torch.compile(m, fullgraph=True, backend="cudagraphs")
        outs += [fn2(x).clone() for _ in range(3)]
    for y in outs:
        assert torch.equal(y, y_eager)


def test_private_scratch_on_a_second_stream():
    # Two streams run layers at the same time: the second one brings its own scratch (the shared per-device buffer
    # holds one launch's intermediate at a time); results equal the single-stream ones bit for bit.
    from nanoquant_b200 import ops
    from nanoquant_b200.modules.linear import NanoQuantLinear
    mods = []
    for i, (n, r, m) in enumerate([(512, 160, 384), (512, 96, 256)]):
        d = oc.synth_linear(n, r, m, 2, seed=70 + i)
        lin = NanoQuantLinear(n, m, r, has_scale_mid=True)
        fill(lin, d)
        lin = lin.cuda()
        lin._prepare_kernel("gemv", DT)
        mods.append(lin)
    x = torch.randn(2, 512, device="cuda").to(DT)
    ref = [m(x).clone() for m in mods]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    mine = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    outs = [None, None]
    for _ in range(20):
        with torch.cuda.stream(side), ops.private_scratch(mine):
            outs[1] = mods[1](x)
        outs[0] = mods[0](x)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], ref[0]) and torch.equal(outs[1], ref[1])
    with pytest.raises(RuntimeError, match="too small"):
        with ops.private_scratch(torch.zeros(64, dtype=torch.uint8, device="cuda")):
            mods[0](x)
