"""B200-native quantized FullyConnected path behind ML Drift's operator surface.

The product is the CUDA library ``libmldfc.so`` (sources in ``csrc/``, C ABI in
``include/mldfc.h``) and the C++ host mirror of the reference interface in
``host/``.  This Python package is a thin ctypes binding over the C ABI for the
tests and the benchmark; it holds no compute of its own and has no CPU
fallback: importing :mod:`binding` fails loudly when the library is missing.
"""
from . import binding, sharding  # noqa: F401
from .binding import *  # noqa: F401,F403
