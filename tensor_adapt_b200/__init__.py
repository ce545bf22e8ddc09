"""tensor_adapt_b200: B200-native (sm_100a) LoRA training hot path of carbon-os/tensor-adapt.

The product is the C-ABI shared library built from csrc/ (see include/tensor_adapt_b200.h);
this package is its ctypes binding plus the host-side mirror used by the tests and bench.py.
"""
from ._lib import Context, TAError, lib, ptr, stream_ptr, exported_symbols, LIB_PATH  # noqa: F401
