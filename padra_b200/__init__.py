"""padra_b200: B200 (sm_100a) kernels for the EXL3 mixture-of-experts expert layer of the Padra server.

The product is the CUDA shared library `libpadra_b200.so` behind the C ABI in include/padra_b200.h.  This
package holds the kernels (csrc/), the in-tree build (build.py) and a ctypes caller (binding.py, experts.py)
used by the tests and the benchmark.  Nothing here computes on the CPU.
"""
from . import binding
from .binding import PadraError, load

__all__ = ["binding", "load", "PadraError"]
