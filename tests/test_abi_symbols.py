"""CPU-only: the library loads and exports every symbol that include/nanoquant_b200.h declares
(no compute calls), and the Python loader's table matches the header."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "nanoquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_loader_binds():
    from nanoquant_b200 import _lib
    syms = header_symbols()
    assert len(syms) >= 20
    assert sorted(_lib.SIGNATURES) == syms


def test_library_exports_every_declared_symbol():
    from nanoquant_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built (python -m nanoquant_b200.build)")
    L = _lib.lib()
    for name in header_symbols():
        assert hasattr(L, name), name
    assert L.nq_abi_version() >= 1
    assert L.nq_strerror(-7).decode().startswith("a bounded")
    # header + four token slots of tagged fp32 (8 bytes per element)
    assert L.nq_gemv_scratch_bytes(1, 4096, 1536, 4096) == 256 + 4 * 1536 * 8
    assert L.nq_tiles_bytes(4096, 1536) == 256 * 6 * 512


def test_operators_register_and_trace_on_cpu():
    import torch
    import binary_kernels  # noqa: F401
    op = torch.ops.binary_kernels.nanoquant_dyn_forward
    with torch._subclasses.FakeTensorMode():
        y = op(torch.empty(3, 64, dtype=torch.float16), torch.empty(64, dtype=torch.float16),
               torch.empty(32, 2, dtype=torch.int32), None, torch.empty(16, 1, dtype=torch.int32),
               torch.empty(16, dtype=torch.float16), num_acc_stage1=1, num_acc_stage2=1)
    assert y.shape == (3, 16)
    for name in ("marlin_onebit_forward", "marlin_nanoquant_forward"):
        assert hasattr(torch.ops.binary_kernels, name)
