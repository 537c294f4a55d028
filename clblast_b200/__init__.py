"""B200-native implementation of CLBlast's GEMM hot path (Gemm, GemmBatched, GemmStridedBatched, Convgemm), of the
level-3 routines built on it (Symm, Hemm, Syrk, Herk, Syr2k, Her2k, Trmm, Trsm) and of the copies either side of it
(Omatcopy, Im2col, Col2im).

The product is ``lib/libclblast.so`` (hand-written sm_100a CUDA kernels behind a C ABI and the reference's C++
API symbols); this package is the Python binding used by the tests and the benchmark.
"""
from .api import (ClearCache, Col2im, Convgemm, Diagonal, FillCache, Gemm, GemmBatched, GemmBatchedStatic,
                  GemmStridedBatched, GemmTempBufferSize, Hemm, Her2k, Herk, Im2col, KernelMode, Layout, Omatcopy,
                  OverrideParameters, Precision, RetrieveParameters, Side, StatusCode, Symm, Syr2k, Syrk, Transpose,
                  Triangle, Trmm, Trsm, last_kernel, launch_count, set_sm_budget, tensor_core_status)
from ._lib import LIB_PATH, LibraryMissing, lib

__all__ = [
    "ClearCache", "Col2im", "Convgemm", "Diagonal", "FillCache", "Gemm", "GemmBatched", "GemmBatchedStatic",
    "GemmStridedBatched", "GemmTempBufferSize", "Hemm", "Her2k", "Herk", "Im2col", "KernelMode", "Layout", "Omatcopy",
    "OverrideParameters", "Precision", "RetrieveParameters", "Side", "StatusCode", "Symm", "Syr2k", "Syrk", "Transpose",
    "Triangle", "Trmm", "Trsm", "last_kernel", "launch_count", "set_sm_budget", "tensor_core_status", "LIB_PATH",
    "LibraryMissing", "lib",
]
