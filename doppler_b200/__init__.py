"""doppler_b200: B200 (sm_100a) implementation of Doppler's Q4_K quantized-inference hot path.

The product is ``libdoppler_b200.so`` (C ABI, ``include/doppler_b200.h``).  This
package is its Python host mirror: :mod:`doppler_b200.ops` restates the
reference's ``src/gpu/kernels/index.js`` op surface, :mod:`doppler_b200.model`
the decode/prefill runner.  There is no CPU fallback.
"""
from ._lib import DopplerError, LIB_PATH, load  # noqa: F401

__all__ = ["DopplerError", "LIB_PATH", "load"]
