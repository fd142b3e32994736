"""B200-native semiring GEMM behind the device-level API of cuASR.

The product is the CUDA library in `csrc/` (C ABI: include/cuasr_b200.h) and the C++ facade in
include/cuasr/.  This Python package is the harness side: a ctypes binding and a mirror of the
reference's `Srgemm` / `SrgemmSplitKParallel` host operators used by the tests and the benchmark.
"""
from .semiring import DType, Layout, Op, RINGS, Status, annihilator, identity  # noqa: F401
from .srgemm import (Arguments, Srgemm, SrgemmSplitKParallel, STATIC_SCRATCH_BYTES, device_status,  # noqa: F401
                     launch_count, pack_k_contiguous, srgemm_path, srgemm_splitk_static)
from .host_pipeline import HostSrgemm  # noqa: F401,E402
