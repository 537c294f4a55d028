"""numpy front end of the CPU oracle (oracle/gemm_oracle.c). TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and bench.py's CPU-baseline legs may import this module; the product package
never does. Function names and arguments follow the reference API, with host numpy arrays in place of device
buffers (half data is carried as numpy float16 arrays).
"""
from __future__ import annotations

import ctypes
import subprocess
from ctypes import c_double, c_int, c_size_t, c_void_p, POINTER
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"

NP_OF = {16: np.float16, 32: np.float32, 64: np.float64, 3232: np.complex64, 6464: np.complex128}
# Error margins of the reference's test harness (test/correctness/tester.cpp:29-69): (relative, absolute).
MARGINS = {16: (0.08, 0.15), 32: (0.005, 0.001), 64: (0.005, 0.001), 3232: (0.005, 0.001), 6464: (0.005, 0.001)}

_lib = None


def build(force: bool = False) -> Path:
    """Compiles liboracle.so with the Makefile next to this file (gcc, OpenMP)."""
    src = HERE / "gemm_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        L = ctypes.CDLL(str(LIB_PATH))
        sz, vp, i = c_size_t, c_void_p, c_int
        L.oracle_gemm.restype = i
        L.oracle_gemm.argtypes = [i, i, i, i, sz, sz, sz, vp, vp, sz, sz, vp, sz, sz, vp, vp, sz, sz]
        L.oracle_gemm_f64.restype = i
        L.oracle_gemm_f64.argtypes = [i, i, i, i, sz, sz, sz, POINTER(c_double), vp, sz, sz, vp, sz, sz,
                                      POINTER(c_double), vp, sz, sz]
        L.oracle_gemm_f64_sampled.restype = i
        L.oracle_gemm_f64_sampled.argtypes = [i, i, i, i, sz, c_double, vp, sz, sz, vp, sz, sz, sz, vp, vp, vp, vp]
        L.oracle_convgemm.restype = i
        L.oracle_convgemm.argtypes = [i, i] + [sz] * 13 + [vp, sz, vp, sz, vp, sz, vp]
        L.oracle_conv_output_size.restype = None
        L.oracle_conv_output_size.argtypes = [sz] * 10 + [POINTER(sz), POINTER(sz)]
        L.oracle_count_mismatches.restype = sz
        L.oracle_count_mismatches.argtypes = [vp, vp, sz, c_double, c_double, POINTER(c_double)]
        _lib = L
    return _lib


def _vp(arr: np.ndarray):
    assert arr.flags["C_CONTIGUOUS"]
    return arr.ctypes.data_as(c_void_p)


def _pair(value):
    v = complex(value)
    return (c_double * 2)(v.real, v.imag)


def widen(precision: int, buf: np.ndarray) -> np.ndarray:
    """The buffer as float64 (complex128 for complex precisions)."""
    return buf.astype(np.complex128 if precision in (3232, 6464) else np.float64)


def gemm(precision, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld):
    """Reference-order GEMM in the routine's own type, in place on the host buffer ``c``."""
    dt = NP_OF[precision]
    al = np.array([alpha], dtype=dt)
    be = np.array([beta], dtype=dt)
    st = lib().oracle_gemm(precision, int(layout), int(ta), int(tb), m, n, k, _vp(al), _vp(a), a_off, a_ld, _vp(b),
                           b_off, b_ld, _vp(be), _vp(c), c_off, c_ld)
    if st != 0:
        raise RuntimeError(f"oracle_gemm failed: {st}")
    return c


def gemm_f64(precision, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld):
    """fp64 yardstick: returns a widened copy of ``c`` updated in place with the exact-order fp64 product."""
    c64 = np.ascontiguousarray(widen(precision, c))
    view = c64.view(np.float64)
    st = lib().oracle_gemm_f64(precision, int(layout), int(ta), int(tb), m, n, k, _pair(alpha), _vp(a), a_off, a_ld,
                               _vp(b), b_off, b_ld, _pair(beta), _vp(view), c_off, c_ld)
    if st != 0:
        raise RuntimeError(f"oracle_gemm_f64 failed: {st}")
    return c64


def gemm_f64_sampled(precision, layout, ta, tb, k, alpha, a, a_off, a_ld, b, b_off, b_ld, rows, cols):
    """(values, magnitudes): alpha*sum_k a*b in fp64 at the sampled (row, col) pairs, and sum_k |a*b|."""
    rows = np.ascontiguousarray(rows, dtype=np.uint64)
    cols = np.ascontiguousarray(cols, dtype=np.uint64)
    out = np.empty(len(rows), dtype=np.float64)
    mag = np.empty(len(rows), dtype=np.float64)
    st = lib().oracle_gemm_f64_sampled(precision, int(layout), int(ta), int(tb), k, float(alpha), _vp(a), a_off, a_ld,
                                       _vp(b), b_off, b_ld, len(rows), _vp(rows), _vp(cols), _vp(out), _vp(mag))
    if st != 0:
        raise RuntimeError(f"oracle_gemm_f64_sampled failed: {st}")
    return out, mag


def conv_output_size(height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w):
    oh, ow = c_size_t(0), c_size_t(0)
    lib().oracle_conv_output_size(height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
                                  ctypes.byref(oh), ctypes.byref(ow))
    return oh.value, ow.value


def convgemm(precision, mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h,
             dil_w, num_kernels, batch_count, im, im_off, ker, ker_off, result, result_off, f64: bool = False):
    """Host convolution in the loop order of the reference's own check. ``f64`` returns a float64 result buffer
    (same geometry as ``result``, untouched entries copied from it); otherwise ``result`` is updated in place."""
    args = [precision, int(mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w,
            dil_h, dil_w, num_kernels, batch_count, _vp(im), im_off, _vp(ker), ker_off]
    if f64:
        out = np.ascontiguousarray(result.astype(np.float64))
        st = lib().oracle_convgemm(*args, None, result_off, _vp(out))
    else:
        out = result
        st = lib().oracle_convgemm(*args, _vp(result), result_off, None)
    if st != 0:
        raise RuntimeError(f"oracle_convgemm failed: {st}")
    return out


def count_mismatches(precision, got: np.ndarray, want: np.ndarray):
    """(failures, max |difference|) under the reference's similarity rule; complex compares re and im separately."""
    rel, ab = MARGINS[precision]
    g = np.ascontiguousarray(widen(precision, got)).view(np.float64).ravel()
    w = np.ascontiguousarray(widen(precision, want)).view(np.float64).ravel()
    assert g.shape == w.shape
    worst = c_double(0.0)
    bad = lib().oracle_count_mismatches(_vp(g), _vp(w), g.size, ab, rel, ctypes.byref(worst))
    return int(bad), worst.value
