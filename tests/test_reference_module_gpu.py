"""The drop-in, proven with the reference's own Python: the reference's ``NanoQuantLinear`` (staged unmodified by
``oracle/make_ref.py``) runs its ``_prepare_kernel`` and kernel ``forward`` (``src/nanoquant/modules/linear.py:106-141,
152-204``) on top of this repository's ``binary_kernels`` operators, and its results match the fp64 oracle and
its own PyTorch branch."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import make_ref
from oracle import nanoquant_oracle as oc
from tests.util import assert_parity, exact_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    pkg = make_ref.load()
    if pkg is None:
        pytest.skip("oracle/_ref not staged (python oracle/make_ref.py needs the reference sources)")
    import importlib
    return importlib.import_module("nanoquant_ref.modules.linear")


def reference_module(ref, d, N, R, M, has_mid=True):
    lin = nn.Linear(N, M, bias=False)
    lin.__class__ = ref.NanoQuantLinear                       # the reference loader's class swap (load_utils.py:319-327)
    lin.init_for_inference(rank=R, has_scale_mid=has_mid)
    with torch.no_grad():
        lin.V.copy_(torch.from_numpy(d["V"]).float())
        lin.U.copy_(torch.from_numpy(d["U"]).float())
        lin.scale_pre.copy_(torch.from_numpy(d["s_pre"]).float()[None])
        if has_mid:
            lin.scale_mid.copy_(torch.from_numpy(d["s_mid"]).float()[None])
        lin.scale_post.copy_(torch.from_numpy(d["s_post"]).float()[None])
    return lin


@pytest.mark.parametrize("kernel_type,T,dtype", [("gemv", 1, torch.float16), ("gemv", 3, torch.bfloat16),
                                                 ("gemm", 96, torch.float16), ("gemm", 300, torch.bfloat16)])
def test_reference_module_runs_on_these_kernels(ref, kernel_type, T, dtype):
    import binary_kernels  # noqa: F401  this repository's operators under the reference's module name
    N, R, M = 1024, 256, 768          # out % 64 == 0, in % 16 == 0, rank % 256 == 0: what the reference's packers accept
    d = oc.synth_linear(N, R, M, T, seed=T)
    lin = reference_module(ref, d, N, R, M).cuda()
    x = torch.from_numpy(d["x"].astype(np.float32)).to(dtype).cuda()
    with torch.no_grad():
        y_torch = lin(x.to(torch.bfloat16))                  # the reference's PyTorch branch (bf16 parameters)
    stance = getattr(torch.compiler, "set_stance", None)     # its packers are @torch.compile'd: run them eagerly
    if stance:
        stance("force_eager")
    try:
        lin._prepare_kernel(kernel_type, dtype)
    finally:
        if stance:
            stance("default")
    assert lin.do_kernel_inference and lin.V_int8.dtype == torch.int32
    with torch.no_grad():
        y = lin(x)
    assert y.shape == (T, M) and y.dtype == dtype
    # the module rounds its scales to bf16 when it is built for inference (linear.py:76,90), then to `dtype`
    sc = lambda a: exact_np(torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).to(dtype))
    y64 = oc.forward_fp64(exact_np(x), d["V"], d["U"], sc(d["s_pre"]), sc(d["s_mid"]), sc(d["s_post"]))
    assert_parity(exact_np(y), y64, dtype, what=f"reference module, {kernel_type}")
    # and its own dense bf16 path agrees with the kernels to bf16 accuracy
    assert oc.rel_err(exact_np(y), exact_np(y_torch)) < 2e-2
