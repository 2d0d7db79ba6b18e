"""miroxen_b200: sm_100a implementation of Miroxen's fused DiT layer ops (src/kernels/ops.h).

The product is ``lib/libmxk.so`` (CUDA kernels + C ABI, declared in ``include/mxk.h``).  This
package is the thin Python host mirror used by the tests and the benchmark: it loads the library
with ctypes and exposes the reference's launcher names on torch tensors.  There is no fallback:
if the library is missing or a call fails, an exception is raised.
"""
from ._lib import MxkError, lib, lib_path  # noqa: F401
from .ops import *  # noqa: F401,F403
