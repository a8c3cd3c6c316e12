"""Generate the golden fixtures in this folder by RUNNING the reference.

Usage (only where the reference checkout is present; the fixtures it writes are
committed, so tests never need the reference at run time)::

    python tests/golden/make_golden.py /path/to/NanoQuant

The reference's Python packers and its quantised-linear module are imported
from ``<reference>/src`` and executed on CPU.  Two shims are needed to import it
in an environment without its optional dependencies: ``TORCHDYNAMO_DISABLE=1``
(the two row packers are wrapped in ``torch.compile``) and stub modules for
``cut_cross_entropy`` and ``lm_eval`` (pulled in by unrelated parts of the
package ``__init__``).

Fixtures (all small, ``.npz``):

* ``pack_rows.npz``      ragged ±1 matrices and their ``lsb_first`` / ``half2`` words
* ``pack_onehot.npz``    single -1 at chosen columns (known-answer words)
* ``pack_marlin.npz``    Marlin-fragment packing incl. scale permutations
* ``pack_marlin_fused.npz`` two-stage fused packer with rank padding
* ``forward_fp64.npz``   the reference module's PyTorch forward, module cast to float64
* ``forward_bf16.npz``   the same forward in the module's own bf16
* ``ranks.npz``          rank-from-bits formula on the workload shapes
"""
import os
import sys
import types

os.environ["TORCHDYNAMO_DISABLE"] = "1"

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    cce = types.ModuleType("cut_cross_entropy")
    cce.linear_cross_entropy = lambda *a, **k: None
    sys.modules.setdefault("cut_cross_entropy", cce)
    lm = types.ModuleType("lm_eval")
    ev = types.ModuleType("lm_eval.evaluator")
    ev.simple_evaluate = lambda *a, **k: None
    lm.evaluator = ev
    sys.modules.setdefault("lm_eval", lm)
    sys.modules.setdefault("lm_eval.evaluator", ev)
    import nanoquant.kernel.utils as ku
    import nanoquant.modules.linear as lin
    import nanoquant.utils.utils as uu
    return ku, lin, uu


def signs(g, shape):
    return (torch.randint(0, 2, shape, generator=g, dtype=torch.int8) * 2 - 1).to(torch.int8)


def main(ref_root):
    ku, lin, uu = import_reference(ref_root)
    g = torch.Generator().manual_seed(0)

    # --- row packers -------------------------------------------------------
    out = {}
    for name, shape in (("a", (5, 32)), ("b", (7, 70)), ("c", (16, 257)), ("d", (1, 1)), ("e", (3, 96))):
        w = signs(g, shape)
        out[f"{name}_w"] = w.numpy()
        for m in ("lsb_first", "half2"):
            p = ku.pack_binary_gemv(w, method=m)
            out[f"{name}_{m}"] = p.numpy()
            back = ku.unpack_binary_gemv(p, shape, method=m)
            assert torch.equal(back, w)
    np.savez_compressed(os.path.join(HERE, "pack_rows.npz"), **out)

    out = {}
    cols = list(range(32)) + [32, 63]
    for m in ("lsb_first", "half2"):
        words = []
        for c in cols:
            w = torch.ones(1, 64, dtype=torch.int8)
            w[0, c] = -1
            words.append(ku.pack_binary_gemv(w, method=m).numpy()[0])
        out[m] = np.stack(words)
    out["cols"] = np.array(cols)
    np.savez_compressed(os.path.join(HERE, "pack_onehot.npz"), **out)

    # --- marlin packers ----------------------------------------------------
    out = {}
    for name, shape in (("a", (128, 32)), ("b", (64, 48)), ("c", (192, 16))):
        w = signs(g, shape)
        s_in = torch.rand(shape[1], generator=g).to(torch.float16)
        s_out = torch.rand(shape[0], generator=g).to(torch.float16)
        # pack_binary_marlin derives the workspace size from scale_out.numel() // 128
        B, si, so, ws = ku.pack_binary_marlin(w, s_in, s_out)
        out[f"{name}_w"] = w.numpy()
        out[f"{name}_s_in"] = s_in.numpy()
        out[f"{name}_s_out"] = s_out.numpy()
        out[f"{name}_B"] = B.numpy()
        out[f"{name}_s_in_p"] = si.numpy()
        out[f"{name}_s_out_p"] = so.numpy()
        out[f"{name}_ws"] = np.array(ws)
    # one-hot known answers on a 128 x 32 matrix
    hot = [(0, 0), (0, 1), (1, 0), (8, 0), (16, 0), (0, 8), (0, 2), (64, 0), (0, 16), (127, 31)]
    hot_B = []
    for (o, i) in hot:
        w = torch.ones(128, 32, dtype=torch.int8)
        w[o, i] = -1
        B, _, _, _ = ku.pack_binary_marlin(w, torch.ones(32), torch.ones(128))
        hot_B.append(B.numpy())
    out["hot_idx"] = np.array(hot)
    out["hot_B"] = np.stack(hot_B)
    np.savez_compressed(os.path.join(HERE, "pack_marlin.npz"), **out)

    out = {}
    N, R, M = 64, 96, 128
    V_sign = signs(g, (N, R))
    U_sign = signs(g, (R, M))
    sg = torch.rand(N, generator=g).to(torch.float16)
    sl = torch.rand(R, generator=g).to(torch.float16)
    sh = torch.rand(M, generator=g).to(torch.float16)
    Vb, Ub, s1, s2, s3, ws = ku.pack_binary_marlin_fused(V_sign, U_sign, sg, sl, sh)
    out.update(V_sign=V_sign.numpy(), U_sign=U_sign.numpy(), sg=sg.numpy(), sl=sl.numpy(), sh=sh.numpy(),
               Vb=Vb.numpy(), Ub=Ub.numpy(), s1=s1.numpy(), s2=s2.numpy(), s3=s3.numpy(), ws=ws.numpy())
    np.savez_compressed(os.path.join(HERE, "pack_marlin_fused.npz"), **out)

    # --- forward -----------------------------------------------------------
    def make_module(N, R, M, has_mid, dtype):
        m = torch.nn.Linear(N, M, bias=False)
        m.__class__ = lin.NanoQuantLinear
        m.init_for_inference(rank=R, has_scale_mid=has_mid)
        m = m.to(dtype)
        V = signs(g, (R, N))
        U = signs(g, (M, R))
        sp = ((torch.rand(1, N, generator=g) + 0.5) * 0.01).to(torch.float16)
        sm = ((torch.rand(1, R, generator=g) + 0.5) * 0.01).to(torch.float16)
        so = ((torch.rand(1, M, generator=g) + 0.5) * 0.01).to(torch.float16)
        with torch.no_grad():
            m.V.copy_(V.to(dtype))
            m.U.copy_(U.to(dtype))
            m.scale_pre.copy_(sp.to(dtype))
            m.scale_post.copy_(so.to(dtype))
            if has_mid:
                m.scale_mid.copy_(sm.to(dtype))
        return m, V, U, sp, sm, so

    out = {}
    for name, (N, R, M, T, has_mid) in {"a": (64, 32, 96, 3, True), "b": (160, 64, 32, 1, False),
                                       "c": (256, 96, 128, 5, True)}.items():
        m, V, U, sp, sm, so = make_module(N, R, M, has_mid, torch.float64)
        x = torch.randn(T, N, generator=g).to(torch.float16)
        with torch.no_grad():
            y = m(x.double())
        out[f"{name}_x"] = x.numpy()
        out[f"{name}_V"] = V.numpy()
        out[f"{name}_U"] = U.numpy()
        out[f"{name}_s_pre"] = sp.numpy()[0]
        out[f"{name}_s_post"] = so.numpy()[0]
        if has_mid:
            out[f"{name}_s_mid"] = sm.numpy()[0]
        out[f"{name}_y"] = y.numpy()
        # the module's own state_dict packs V/U in the checkpoint (lsb_first) layout
        sd = m.state_dict()
        out[f"{name}_V_packed"] = sd["V_packed"].numpy()
        out[f"{name}_U_packed"] = sd["U_packed"].numpy()
        out[f"{name}_V_shape"] = sd["V_shape"].numpy()
        out[f"{name}_U_shape"] = sd["U_shape"].numpy()
    np.savez_compressed(os.path.join(HERE, "forward_fp64.npz"), **out)

    out = {}
    N, R, M, T = 128, 64, 96, 4
    m, V, U, sp, sm, so = make_module(N, R, M, True, torch.bfloat16)
    x = torch.randn(T, N, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        y = m(x)
    # bf16 has no numpy dtype: store the exact values widened to float32
    out.update(x=x.float().numpy(), V=V.numpy(), U=U.numpy(),
               s_pre=m.scale_pre.float().numpy()[0], s_mid=m.scale_mid.float().numpy()[0],
               s_post=m.scale_post.float().numpy()[0], y=y.float().numpy())
    np.savez_compressed(os.path.join(HERE, "forward_bf16.npz"), **out)

    # --- ranks -------------------------------------------------------------
    # calculate_ranks walks model.model.layers[i].<name>; a one-block stand-in is enough
    shapes = [(4096, 4096, 0.75), (2048, 2048, 1.0), (2048, 512, 1.0), (2048, 8192, 1.0), (8192, 2048, 1.0),
              (4096, 4096, 0.8), (4096, 1024, 0.8), (4096, 12288, 0.8), (12288, 4096, 0.8),
              (4096, 4096, 1.0), (4096, 11008, 1.0), (11008, 4096, 1.0),
              (8192, 8192, 0.8), (8192, 1024, 0.8), (8192, 28672, 0.8), (28672, 8192, 0.8)]
    rows = []
    for (a, b, bits) in shapes:
        for admm, ns in (("nanoquant", 2), ("dbf", 3)):
            lx = torch.nn.Linear(1, 1, bias=False)
            lx.in_features, lx.out_features = a, b
            block = torch.nn.Module()
            block.proj = lx
            model = torch.nn.Module()
            model.config = types.SimpleNamespace(model_type="llama")
            model.model = torch.nn.Module()
            model.model.layers = torch.nn.ModuleList([block])
            r = uu.calculate_ranks(model, ["proj"], {"bits": bits, "admm_type": admm})
            rows.append((a, b, bits, ns, r["0.proj"]))
    np.savez_compressed(os.path.join(HERE, "ranks.npz"), table=np.array(rows, dtype=np.float64))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of SamsungLabs/NanoQuant>")
    main(sys.argv[1])
