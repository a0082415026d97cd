"""beholdd_b200: B200-native (sm_100a) quantised matvec / matmul and qwen3moe routed-expert
layer behind beholdd's `Device` operator interface.

The arithmetic lives in `libbeholdd_b200.so` (hand-written CUDA behind the C ABI declared in
include/beholdd_b200.h). This package is the host-side mirror of the reference interface and
the seeded input generators; it contains no CPU implementation of the path.
"""
from . import synth  # noqa: F401
from .device import (AllocationError, BackendError, CudaDevice, DeviceError, ResidentWeight, ShapeError,  # noqa: F401
                     UnsupportedFormat, Weight, load_library, LIB_PATH, EXPORTS)

F32, F16, Q8_0, Q4_K, Q5_K, Q6_K = 0, 1, 8, 12, 13, 14
