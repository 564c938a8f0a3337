"""morok_b200 -- a B200 (sm_100a) device for the dense hot path of npatsakula/morok.

The product is `libmorok_b200.so` (C ABI in include/morok_b200.h).  This package holds its CUDA
sources (csrc/), the build driver and a thin ctypes layer used by the tests and the benchmark.
"""
from ._ffi import (MK_BF16, MK_BOOL, MK_F16, MK_F32, MK_F8E4M3, MK_F8E5M2, MorokError, load)  # noqa: F401
from .device import Buffer, Device, Event, Stream, device_count, dtype_size  # noqa: F401
from .tensor import Plan, Tensor  # noqa: F401,E402
