"""The library's measurement probes answer with plausible figures and reject bad arguments (they are what
``bench.py --mode probe`` prints; nothing on the hot path calls them)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_probes_run_and_check_their_arguments():
    from nanoquant_b200 import _lib
    L = _lib.lib()
    torch.zeros(1, device="cuda")
    out = ctypes.c_float()
    assert L.nq_probe_chain(37, 512, 0, ctypes.byref(out)) == 0
    assert 0.5 < out.value < 50.0            # microseconds per launch
    assert L.nq_probe_chain(0, 512, 0, ctypes.byref(out)) == _lib.NQ_ERR_SHAPE
    assert L.nq_probe_chain(37, 511, 0, ctypes.byref(out)) == _lib.NQ_ERR_SHAPE
    assert L.nq_probe_chain(37, 512, 0, None) == _lib.NQ_ERR_NULL
    for mode in (0, 1, 2):
        assert L.nq_probe_loop(mode, 16, ctypes.byref(out)) == 0
        assert out.value > 100.0             # GB/s
    assert L.nq_probe_loop(3, 16, ctypes.byref(out)) == _lib.NQ_ERR_SHAPE
    assert L.nq_probe_loop(0, 6, ctypes.byref(out)) == _lib.NQ_ERR_SHAPE
