"""Python mirror of the reference's CUDA API for the GEMM family, over the library's C ABI.

Function names, argument order and meaning and the returned status codes are those of the reference's
``include/clblast_cuda.h`` (Gemm :385-390, Convgemm :486-493, GemmBatched :502-507, GemmStridedBatched :511-518,
GemmTempBufferSize :523-527, cache and parameter calls :533-550), so the parity tests read like the reference's own
test descriptors (``test/routines/level3/xgemm.hpp:115-121``). Buffers are device pointers (``int``) or CUDA
``torch.Tensor`` objects; the element type comes from ``precision`` or, for tensors, from the tensor's dtype.
``context``/``device`` of the C++ signature are implicit: the calling thread's current CUDA context is used.

Every call returns a :class:`StatusCode` value; nothing is computed on the host, and a missing library raises.
"""
from __future__ import annotations

import ctypes
import enum
import struct
from typing import Sequence

import numpy as np

from ._lib import lib


class StatusCode(enum.IntEnum):
    kSuccess = 0
    kNotImplemented = -1024
    kInvalidMatrixA = -1022
    kInvalidMatrixB = -1021
    kInvalidMatrixC = -1020
    kInvalidDimension = -1017
    kInvalidLeadDimA = -1016
    kInvalidLeadDimB = -1015
    kInvalidLeadDimC = -1014
    kInsufficientMemoryA = -1011
    kInsufficientMemoryB = -1010
    kInsufficientMemoryC = -1009
    kInsufficientMemoryTemp = -2050
    kInvalidBatchCount = -2049
    kInvalidOverrideKernel = -2048
    kMissingOverrideParameter = -2047
    kNoHalfPrecision = -2045
    kNoDoublePrecision = -2044
    kDatabaseError = -2041
    kUnknownError = -2040
    kUnexpectedError = -2039


class Layout(enum.IntEnum):
    kRowMajor = 101
    kColMajor = 102


class Transpose(enum.IntEnum):
    kNo = 111
    kYes = 112
    kConjugate = 113


class Triangle(enum.IntEnum):
    kUpper = 121
    kLower = 122


class Diagonal(enum.IntEnum):
    kNonUnit = 131
    kUnit = 132


class Side(enum.IntEnum):
    kLeft = 141
    kRight = 142


class KernelMode(enum.IntEnum):
    kCrossCorrelation = 151
    kConvolution = 152


class Precision(enum.IntEnum):
    kHalf = 16
    kSingle = 32
    kDouble = 64
    kComplexSingle = 3232
    kComplexDouble = 6464


_NP_OF = {16: np.float16, 32: np.float32, 64: np.float64, 3232: np.complex64, 6464: np.complex128}


def precision_of(buf, precision=None) -> int:
    """Precision code of a buffer: explicit, or inferred from a torch tensor's dtype."""
    if precision is not None:
        return int(precision)
    import torch
    table = {torch.float16: 16, torch.float32: 32, torch.float64: 64, torch.complex64: 3232, torch.complex128: 6464}
    if not hasattr(buf, "dtype") or buf.dtype not in table:
        raise TypeError("pass precision= for raw pointers or unsupported tensor dtypes")
    return table[buf.dtype]


def _ptr(buf) -> int:
    if buf is None:
        return 0
    if isinstance(buf, int):
        return buf
    if hasattr(buf, "data_ptr"):
        if not buf.is_cuda:
            raise ValueError("buffers must live in device memory")
        return buf.data_ptr()
    raise TypeError(f"unsupported buffer type {type(buf)}")


def scalar_bytes(precision: int, value) -> ctypes.Array:
    """One host scalar of the given precision, laid out as the C ABI expects."""
    if precision == 16:
        raw = np.float16(value).tobytes()
    elif precision in (32, 64):
        raw = _NP_OF[precision](value).tobytes()
    else:
        raw = _NP_OF[precision](complex(value)).tobytes()
    return ctypes.create_string_buffer(raw, len(raw))


def _stream_arg(stream):
    """(pointer, async flag): stream=None reproduces the reference's host-synchronous call."""
    if stream is None:
        return None, 0
    if isinstance(stream, int):
        return ctypes.c_void_p(stream), 1
    return ctypes.c_void_p(stream.cuda_stream), 1


def _status(code: int):
    try:
        return StatusCode(code)
    except ValueError:
        return code  # positive values are raw CUDA error numbers


def Gemm(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta,
         c_buffer, c_offset, c_ld, *, precision=None, stream=None):
    """C = alpha*op(A)*op(B) + beta*C (reference: clblast::Gemm, include/clblast_cuda.h:385-390)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_gemm(p, int(layout), int(a_transpose), int(b_transpose), m, n, k,
                                       scalar_bytes(p, alpha), _ptr(a_buffer), a_offset, a_ld, _ptr(b_buffer),
                                       b_offset, b_ld, scalar_bytes(p, beta), _ptr(c_buffer), c_offset, c_ld, sp,
                                       is_async))


def GemmStridedBatched(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld, a_stride, b_buffer,
                       b_offset, b_ld, b_stride, beta, c_buffer, c_offset, c_ld, c_stride, batch_count, *,
                       precision=None, stream=None):
    """Batch b uses offset + b*stride (reference: clblast::GemmStridedBatched, include/clblast_cuda.h:511-518)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_gemm_strided_batched(
        p, int(layout), int(a_transpose), int(b_transpose), m, n, k, scalar_bytes(p, alpha), _ptr(a_buffer), a_offset,
        a_ld, a_stride, _ptr(b_buffer), b_offset, b_ld, b_stride, scalar_bytes(p, beta), _ptr(c_buffer), c_offset,
        c_ld, c_stride, batch_count, sp, is_async))


def GemmBatched(layout, a_transpose, b_transpose, m, n, k, alphas: Sequence, a_buffer, a_offsets: Sequence[int], a_ld,
                b_buffer, b_offsets: Sequence[int], b_ld, betas: Sequence, c_buffer, c_offsets: Sequence[int], c_ld,
                batch_count, *, precision=None, stream=None):
    """Per-batch scalars and offsets are host sequences (reference: clblast::GemmBatched, clblast_cuda.h:502-507)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    npdt = _NP_OF[p]
    al = np.ascontiguousarray(np.asarray(alphas, dtype=npdt))
    be = np.ascontiguousarray(np.asarray(betas, dtype=npdt))
    if len(al) != batch_count or len(be) != batch_count or len(a_offsets) != batch_count or \
            len(b_offsets) != batch_count or len(c_offsets) != batch_count:
        return StatusCode.kInvalidBatchCount  # the reference checks the vector lengths (xgemmbatched.cpp:70-73)
    arr = ctypes.c_size_t * max(batch_count, 1)
    ao, bo, co = arr(*a_offsets), arr(*b_offsets), arr(*c_offsets)
    return _status(lib().b200blas_gemm_batched(
        p, int(layout), int(a_transpose), int(b_transpose), m, n, k, al.ctypes.data_as(ctypes.c_void_p),
        _ptr(a_buffer), ao, a_ld, _ptr(b_buffer), bo, b_ld, be.ctypes.data_as(ctypes.c_void_p), _ptr(c_buffer), co,
        c_ld, batch_count, sp, is_async))


STATIC_MAX_BATCHES = 4096


def GemmBatchedStatic(layout, a_transpose, b_transpose, m, n, k, alphas: Sequence, a_buffer, a_offsets: Sequence[int],
                      a_ld, b_buffer, b_offsets: Sequence[int], b_ld, betas: Sequence, c_buffer,
                      c_offsets: Sequence[int], c_ld, batch_count, *, stream, wait=True, precision=None):
    """GemmBatched for callers that cannot allocate device memory (a process whose arena owns the whole GPU, a
    latency-critical loop): the per-batch tables live in a fixed array inside the library, so at most
    ``STATIC_MAX_BATCHES`` batches per call, calls on one GPU must not overlap, and the work always runs on the
    caller's ``stream`` (``wait`` synchronises it). No counterpart in the reference."""
    p = precision_of(c_buffer, precision)
    npdt = _NP_OF[p]
    al = np.ascontiguousarray(np.asarray(alphas, dtype=npdt))
    be = np.ascontiguousarray(np.asarray(betas, dtype=npdt))
    if len(al) != batch_count or len(be) != batch_count or len(a_offsets) != batch_count or \
            len(b_offsets) != batch_count or len(c_offsets) != batch_count:
        return StatusCode.kInvalidBatchCount
    arr = ctypes.c_size_t * max(batch_count, 1)
    ao, bo, co = arr(*a_offsets), arr(*b_offsets), arr(*c_offsets)
    sp = ctypes.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream)
    return _status(lib().b200blas_gemm_batched_static(
        p, int(layout), int(a_transpose), int(b_transpose), m, n, k, al.ctypes.data_as(ctypes.c_void_p),
        _ptr(a_buffer), ao, a_ld, _ptr(b_buffer), bo, b_ld, be.ctypes.data_as(ctypes.c_void_p), _ptr(c_buffer), co,
        c_ld, batch_count, sp, 1 if wait else 0))


def Convgemm(kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h,
             dilation_w, num_kernels, batch_count, im_buffer, im_offset, kernel_buffer, kernel_offset, result_buffer,
             result_offset, *, precision=None, stream=None):
    """Batched NCHW convolution (reference: clblast::Convgemm, include/clblast_cuda.h:486-493)."""
    p = precision_of(result_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_convgemm(
        p, int(kernel_mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
        dilation_h, dilation_w, num_kernels, batch_count, _ptr(im_buffer), im_offset, _ptr(kernel_buffer),
        kernel_offset, _ptr(result_buffer), result_offset, sp, is_async))


def _real_precision(p: int) -> int:
    return {3232: 32, 6464: 64}[p]


def Symm(layout, side, triangle, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta, c_buffer,
         c_offset, c_ld, *, precision=None, stream=None, hermitian=False):
    """C = alpha*A*B + beta*C or alpha*B*A + beta*C with A symmetric (reference: clblast::Symm, clblast_cuda.h:393-398)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    fn = lib().b200blas_hemm if hermitian else lib().b200blas_symm
    return _status(fn(p, int(layout), int(side), int(triangle), m, n, scalar_bytes(p, alpha), _ptr(a_buffer), a_offset,
                      a_ld, _ptr(b_buffer), b_offset, b_ld, scalar_bytes(p, beta), _ptr(c_buffer), c_offset, c_ld, sp,
                      is_async))


def Hemm(layout, side, triangle, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta, c_buffer,
         c_offset, c_ld, *, precision=None, stream=None):
    """Symm for a hermitian A (reference: clblast::Hemm, clblast_cuda.h:401-406)."""
    return Symm(layout, side, triangle, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta, c_buffer,
                c_offset, c_ld, precision=precision, stream=stream, hermitian=True)


def Syrk(layout, triangle, a_transpose, n, k, alpha, a_buffer, a_offset, a_ld, beta, c_buffer, c_offset, c_ld, *,
         precision=None, stream=None):
    """One triangle of C = alpha*A*A^T + beta*C (reference: clblast::Syrk, clblast_cuda.h:409-413)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_syrk(p, int(layout), int(triangle), int(a_transpose), n, k, scalar_bytes(p, alpha),
                                       _ptr(a_buffer), a_offset, a_ld, scalar_bytes(p, beta), _ptr(c_buffer), c_offset,
                                       c_ld, sp, is_async))


def Herk(layout, triangle, a_transpose, n, k, alpha, a_buffer, a_offset, a_ld, beta, c_buffer, c_offset, c_ld, *,
         precision=None, stream=None):
    """One triangle of C = alpha*A*A^H + beta*C, alpha and beta real (reference: clblast::Herk, clblast_cuda.h:416-420)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    rp = _real_precision(p)
    return _status(lib().b200blas_herk(p, int(layout), int(triangle), int(a_transpose), n, k, scalar_bytes(rp, alpha),
                                       _ptr(a_buffer), a_offset, a_ld, scalar_bytes(rp, beta), _ptr(c_buffer), c_offset,
                                       c_ld, sp, is_async))


def Syr2k(layout, triangle, ab_transpose, n, k, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta,
          c_buffer, c_offset, c_ld, *, precision=None, stream=None):
    """One triangle of C = alpha*A*B^T + alpha*B*A^T + beta*C (reference: clblast::Syr2k, clblast_cuda.h:423-428)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_syr2k(p, int(layout), int(triangle), int(ab_transpose), n, k, scalar_bytes(p, alpha),
                                        _ptr(a_buffer), a_offset, a_ld, _ptr(b_buffer), b_offset, b_ld,
                                        scalar_bytes(p, beta), _ptr(c_buffer), c_offset, c_ld, sp, is_async))


def Her2k(layout, triangle, ab_transpose, n, k, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta,
          c_buffer, c_offset, c_ld, *, precision=None, stream=None):
    """One triangle of C = alpha*A*B^H + conj(alpha)*B*A^H + beta*C, beta real (reference: clblast::Her2k,
    clblast_cuda.h:431-436)."""
    p = precision_of(c_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_her2k(p, int(layout), int(triangle), int(ab_transpose), n, k, scalar_bytes(p, alpha),
                                        _ptr(a_buffer), a_offset, a_ld, _ptr(b_buffer), b_offset, b_ld,
                                        scalar_bytes(_real_precision(p), beta), _ptr(c_buffer), c_offset, c_ld, sp,
                                        is_async))


def Trmm(layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld,
         *, precision=None, stream=None):
    """B = alpha*op(A)*B or alpha*B*op(A), A triangular (reference: clblast::Trmm, clblast_cuda.h:439-443)."""
    p = precision_of(b_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_trmm(p, int(layout), int(side), int(triangle), int(a_transpose), int(diagonal), m, n,
                                       scalar_bytes(p, alpha), _ptr(a_buffer), a_offset, a_ld, _ptr(b_buffer), b_offset,
                                       b_ld, sp, is_async))


def Trsm(layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld,
         *, precision=None, stream=None):
    """Solves op(A)*X = alpha*B or X*op(A) = alpha*B; X overwrites B (reference: clblast::Trsm, clblast_cuda.h:446-450)."""
    p = precision_of(b_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_trsm(p, int(layout), int(side), int(triangle), int(a_transpose), int(diagonal), m, n,
                                       scalar_bytes(p, alpha), _ptr(a_buffer), a_offset, a_ld, _ptr(b_buffer), b_offset,
                                       b_ld, sp, is_async))


def Omatcopy(layout, a_transpose, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, *, precision=None,
             stream=None):
    """B = alpha*op(A), out of place (reference: clblast::Omatcopy, clblast_cuda.h:464-467)."""
    p = precision_of(b_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_omatcopy(p, int(layout), int(a_transpose), m, n, scalar_bytes(p, alpha), _ptr(a_buffer),
                                           a_offset, a_ld, _ptr(b_buffer), b_offset, b_ld, sp, is_async))


def Im2col(kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h,
           dilation_w, im_buffer, im_offset, col_buffer, col_offset, *, precision=None, stream=None):
    """Column matrix of one image (reference: clblast::Im2col, clblast_cuda.h:470-475)."""
    p = precision_of(col_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_im2col(p, int(kernel_mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w,
                                         stride_h, stride_w, dilation_h, dilation_w, _ptr(im_buffer), im_offset,
                                         _ptr(col_buffer), col_offset, sp, is_async))


def Col2im(kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h,
           dilation_w, col_buffer, col_offset, im_buffer, im_offset, *, precision=None, stream=None):
    """Adds the column entries back to the image pixels they came from (reference: clblast::Col2im,
    clblast_cuda.h:478-483)."""
    p = precision_of(im_buffer, precision)
    sp, is_async = _stream_arg(stream)
    return _status(lib().b200blas_col2im(p, int(kernel_mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w,
                                         stride_h, stride_w, dilation_h, dilation_w, _ptr(col_buffer), col_offset,
                                         _ptr(im_buffer), im_offset, sp, is_async))


def GemmTempBufferSize(layout, a_transpose, b_transpose, m, n, k, a_offset, a_ld, b_offset, b_ld, c_offset, c_ld, *,
                       precision):
    """(status, bytes) — always 0 bytes here (reference: clblast::GemmTempBufferSize, clblast_cuda.h:523-527)."""
    out = ctypes.c_size_t(0)
    st = lib().b200blas_gemm_temp_buffer_size(int(precision), int(layout), int(a_transpose), int(b_transpose), m, n, k,
                                              a_offset, a_ld, b_offset, b_ld, c_offset, c_ld, ctypes.byref(out))
    return _status(st), out.value


def ClearCache():
    return _status(lib().b200blas_clear_cache())


def FillCache(device: int = 0):
    return _status(lib().b200blas_fill_cache(device))


def OverrideParameters(device: int, kernel_name: str, precision, parameters: dict):
    names = list(parameters.keys())
    n = len(names)
    c_names = (ctypes.c_char_p * max(n, 1))(*[s.encode() for s in names])
    c_vals = (ctypes.c_size_t * max(n, 1))(*[int(parameters[s]) for s in names])
    return _status(lib().b200blas_override_parameters(device, kernel_name.encode(), int(precision), c_names, c_vals, n))


def RetrieveParameters(device: int, kernel_name: str, precision):
    """(status, dict) of the family's current parameter values."""
    count = ctypes.c_size_t(0)
    st = lib().b200blas_retrieve_parameters(device, kernel_name.encode(), int(precision), None, None, 0,
                                            ctypes.byref(count))
    if st != 0:
        return _status(st), {}
    n = count.value
    c_names = (ctypes.c_char_p * n)()
    c_vals = (ctypes.c_size_t * n)()
    st = lib().b200blas_retrieve_parameters(device, kernel_name.encode(), int(precision), c_names, c_vals, n,
                                            ctypes.byref(count))
    return _status(st), {c_names[i].decode(): c_vals[i] for i in range(n)}


def set_sm_budget(sms: int) -> None:
    """Limits how many SMs the persistent tensor-core kernels occupy (0 = all), e.g. to leave room for a collective."""
    lib().b200blas_set_sm_budget(int(sms))


def tensor_core_status(clear: bool = True):
    """(status, [code, block, barrier, 0]) of the tensor-core kernels' bounded waits; for callers that enqueue on their
    own stream, after synchronising it. status is kUnexpectedError when a wait expired since the last clear."""
    out = (ctypes.c_uint * 4)()
    st = lib().b200blas_tensor_core_status(out, 1 if clear else 0)
    return _status(st), list(out)


def last_kernel() -> str:
    """Kernel family chosen by the most recent compute call on this thread."""
    return lib().b200blas_last_kernel().decode()


def launch_count() -> int:
    return int(lib().b200blas_launch_count())
