"""Drop-in for the reference's compiled ``binary_kernels`` extension module.

Importing it registers ``torch.ops.binary_kernels.*`` (same schemas as the
reference's ``src/nanoquant/kernel/pybind.cpp:83-105``) on top of
``libnanoquant_b200.so``.  The reference imports this module by name
(``src/nanoquant/kernel/utils.py:35``, ``src/nanoquant/modules/linear.py:201``).
"""
from nanoquant_b200 import _lib as _lib
from nanoquant_b200 import ops as _ops

_lib.lib()  # fail at import time, loudly, if the CUDA library has not been built
_ops.define_ops()
