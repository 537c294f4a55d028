"""ctypes binding of libclblast.so's C ABI (include/b200blas.h)."""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_size_t, c_uint64, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libclblast.so"

_lib = None


class LibraryMissing(RuntimeError):
    """libclblast.so has not been built; there is no fallback path."""


def lib() -> ctypes.CDLL:
    """Loads the shared library once. Raises LibraryMissing when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise LibraryMissing(f"{LIB_PATH} not found: run `python -m clblast_b200.build` (needs nvcc). "
                             "This package has no CPU or PyTorch fallback.")
    L = ctypes.CDLL(str(LIB_PATH))
    sz, vp, i = c_size_t, c_void_p, c_int
    L.b200blas_gemm.restype = i
    L.b200blas_gemm.argtypes = [i, i, i, i, sz, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, vp, sz, sz, vp, i]
    L.b200blas_gemm_strided_batched.restype = i
    L.b200blas_gemm_strided_batched.argtypes = [i, i, i, i, sz, sz, sz, vp, vp, sz, sz, sz, vp, sz, sz, sz, vp, vp, sz,
                                                sz, sz, sz, vp, i]
    L.b200blas_gemm_batched.restype = i
    L.b200blas_gemm_batched.argtypes = [i, i, i, i, sz, sz, sz, vp, vp, POINTER(sz), sz, vp, POINTER(sz), sz, vp, vp,
                                        POINTER(sz), sz, sz, vp, i]
    L.b200blas_gemm_batched_static.restype = i
    L.b200blas_gemm_batched_static.argtypes = L.b200blas_gemm_batched.argtypes
    L.b200blas_convgemm.restype = i
    L.b200blas_convgemm.argtypes = [i, i] + [sz] * 13 + [vp, sz, vp, sz, vp, sz, vp, i]
    for name in ("b200blas_symm", "b200blas_hemm"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [i, i, i, i, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, vp, sz, sz, vp, i]
    for name in ("b200blas_syrk", "b200blas_herk"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [i, i, i, i, sz, sz, vp, vp, sz, sz, vp, vp, sz, sz, vp, i]
    for name in ("b200blas_syr2k", "b200blas_her2k"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [i, i, i, i, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, vp, sz, sz, vp, i]
    for name in ("b200blas_trmm", "b200blas_trsm"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [i, i, i, i, i, i, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, i]
    L.b200blas_omatcopy.restype = i
    L.b200blas_omatcopy.argtypes = [i, i, i, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, i]
    for name in ("b200blas_im2col", "b200blas_col2im"):
        f = getattr(L, name)
        f.restype = i
        f.argtypes = [i, i] + [sz] * 11 + [vp, sz, vp, sz, vp, i]
    L.b200blas_gemm_temp_buffer_size.restype = i
    L.b200blas_gemm_temp_buffer_size.argtypes = [i, i, i, i] + [sz] * 9 + [POINTER(sz)]
    L.b200blas_clear_cache.restype = i
    L.b200blas_clear_cache.argtypes = []
    L.b200blas_fill_cache.restype = i
    L.b200blas_fill_cache.argtypes = [i]
    L.b200blas_override_parameters.restype = i
    L.b200blas_override_parameters.argtypes = [i, c_char_p, i, POINTER(c_char_p), POINTER(sz), sz]
    L.b200blas_retrieve_parameters.restype = i
    L.b200blas_retrieve_parameters.argtypes = [i, c_char_p, i, POINTER(c_char_p), POINTER(sz), sz, POINTER(sz)]
    L.b200blas_set_sm_budget.restype = None
    L.b200blas_set_sm_budget.argtypes = [i]
    u8p = POINTER(ctypes.c_ubyte)
    L.b200blas_ipc_export.restype = i
    L.b200blas_ipc_export.argtypes = [vp, u8p, POINTER(sz)]
    L.b200blas_ipc_open.restype = i
    L.b200blas_ipc_open.argtypes = [u8p, sz, POINTER(vp)]
    L.b200blas_ipc_close.restype = i
    L.b200blas_ipc_close.argtypes = [vp, sz]
    L.b200blas_stream_copy.restype = i
    L.b200blas_stream_copy.argtypes = [vp, vp, vp, sz]
    L.b200blas_stream_wait_flag.restype = i
    L.b200blas_stream_wait_flag.argtypes = [vp, vp, ctypes.c_uint32]
    L.b200blas_stream_write_flag.restype = i
    L.b200blas_stream_write_flag.argtypes = [vp, vp, ctypes.c_uint32]
    L.b200blas_tensor_core_status.restype = i
    L.b200blas_tensor_core_status.argtypes = [POINTER(ctypes.c_uint), i]
    L.b200blas_last_kernel.restype = c_char_p
    L.b200blas_last_kernel.argtypes = []
    L.b200blas_launch_count.restype = c_uint64
    L.b200blas_launch_count.argtypes = []
    L.b200blas_version.restype = c_char_p
    L.b200blas_version.argtypes = []
    _lib = L
    return L


# Every symbol include/b200blas.h declares; tests check that the built library exports all of them.
C_ABI_SYMBOLS = [
    "b200blas_gemm", "b200blas_gemm_strided_batched", "b200blas_gemm_batched", "b200blas_gemm_batched_static",
    "b200blas_convgemm", "b200blas_symm", "b200blas_hemm", "b200blas_syrk", "b200blas_herk", "b200blas_syr2k",
    "b200blas_her2k", "b200blas_trmm", "b200blas_trsm", "b200blas_omatcopy", "b200blas_im2col", "b200blas_col2im",
    "b200blas_gemm_temp_buffer_size", "b200blas_clear_cache", "b200blas_fill_cache", "b200blas_override_parameters",
    "b200blas_retrieve_parameters", "b200blas_set_sm_budget", "b200blas_tensor_core_status", "b200blas_ipc_export", "b200blas_ipc_open",
    "b200blas_ipc_close", "b200blas_stream_copy", "b200blas_stream_wait_flag", "b200blas_stream_write_flag", "b200blas_last_kernel", "b200blas_launch_count", "b200blas_version",
]

# Every symbol include/b200blas_c.h and include/b200blas_netlib.h declare.
C_API_SYMBOLS = ['CLBlastSgemm', 'CLBlastDgemm', 'CLBlastCgemm', 'CLBlastZgemm', 'CLBlastHgemm', 'CLBlastSsymm', 'CLBlastDsymm', 'CLBlastCsymm', 'CLBlastZsymm', 'CLBlastHsymm', 'CLBlastChemm', 'CLBlastZhemm', 'CLBlastSsyrk', 'CLBlastDsyrk', 'CLBlastCsyrk', 'CLBlastZsyrk', 'CLBlastHsyrk', 'CLBlastCherk', 'CLBlastZherk', 'CLBlastSsyr2k', 'CLBlastDsyr2k', 'CLBlastCsyr2k', 'CLBlastZsyr2k', 'CLBlastHsyr2k', 'CLBlastCher2k', 'CLBlastZher2k', 'CLBlastStrmm', 'CLBlastDtrmm', 'CLBlastCtrmm', 'CLBlastZtrmm', 'CLBlastHtrmm', 'CLBlastStrsm', 'CLBlastDtrsm', 'CLBlastCtrsm', 'CLBlastZtrsm', 'CLBlastSomatcopy', 'CLBlastDomatcopy', 'CLBlastComatcopy', 'CLBlastZomatcopy', 'CLBlastHomatcopy', 'CLBlastSim2col', 'CLBlastDim2col', 'CLBlastCim2col', 'CLBlastZim2col', 'CLBlastHim2col', 'CLBlastScol2im', 'CLBlastDcol2im', 'CLBlastCcol2im', 'CLBlastZcol2im', 'CLBlastHcol2im', 'CLBlastSconvgemm', 'CLBlastDconvgemm', 'CLBlastHconvgemm', 'CLBlastSgemmBatched', 'CLBlastDgemmBatched', 'CLBlastCgemmBatched', 'CLBlastZgemmBatched', 'CLBlastHgemmBatched', 'CLBlastSgemmStridedBatched', 'CLBlastDgemmStridedBatched', 'CLBlastCgemmStridedBatched', 'CLBlastZgemmStridedBatched', 'CLBlastHgemmStridedBatched']
NETLIB_SYMBOLS = ['cblas_sgemm', 'cblas_dgemm', 'cblas_cgemm', 'cblas_zgemm', 'cblas_ssymm', 'cblas_dsymm', 'cblas_csymm', 'cblas_zsymm', 'cblas_chemm', 'cblas_zhemm', 'cblas_ssyrk', 'cblas_dsyrk', 'cblas_csyrk', 'cblas_zsyrk', 'cblas_cherk', 'cblas_zherk', 'cblas_ssyr2k', 'cblas_dsyr2k', 'cblas_csyr2k', 'cblas_zsyr2k', 'cblas_cher2k', 'cblas_zher2k', 'cblas_strmm', 'cblas_dtrmm', 'cblas_ctrmm', 'cblas_ztrmm', 'cblas_strsm', 'cblas_dtrsm', 'cblas_ctrsm', 'cblas_ztrsm', 'cblas_somatcopy', 'cblas_domatcopy', 'cblas_comatcopy', 'cblas_zomatcopy']
