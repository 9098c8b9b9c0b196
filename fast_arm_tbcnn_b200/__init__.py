"""B200 (sm_100a) implementation of the fast-arm-tbcnn hot path.

The product is the CUDA library ``lib/libtbn_cuda.so`` (C ABI: ``include/tbn_cuda.h``)
and the C++ host layer mirroring the reference's ``tbn::`` API (``host/``).  This Python
package is the ctypes binding used by the tests and the benchmark; it has no CPU fallback
and raises if the library is missing.
"""
from .capi import TbnError, lib, load  # noqa: F401
