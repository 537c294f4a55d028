"""B200-native implementation of CLBlast's GEMM hot path (Gemm, GemmBatched, GemmStridedBatched, Convgemm).

The product is ``lib/libclblast.so`` (hand-written sm_100a CUDA kernels behind a C ABI and the reference's C++
API symbols); this package is the Python binding used by the tests and the benchmark.
"""
from .api import (ClearCache, Convgemm, FillCache, Gemm, GemmBatched, GemmBatchedStatic, GemmStridedBatched, GemmTempBufferSize,
                  KernelMode, Layout, OverrideParameters, Precision, RetrieveParameters, StatusCode, Transpose,
                  last_kernel, launch_count, set_sm_budget, tensor_core_status)
from ._lib import LIB_PATH, LibraryMissing, lib

__all__ = [
    "ClearCache", "Convgemm", "FillCache", "Gemm", "GemmBatched", "GemmBatchedStatic", "GemmStridedBatched", "GemmTempBufferSize",
    "KernelMode", "Layout", "OverrideParameters", "Precision", "RetrieveParameters", "StatusCode", "Transpose",
    "last_kernel", "launch_count", "set_sm_budget", "tensor_core_status", "LIB_PATH", "LibraryMissing", "lib",
]
