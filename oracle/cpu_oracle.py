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
    newest = max((HERE / f).stat().st_mtime for f in ("gemm_oracle.c", "level3_oracle.c", "Makefile"))
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
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
        dp = POINTER(c_double)
        L.oracle_expand_triangle.restype = i
        L.oracle_expand_triangle.argtypes = [i, i, i, i, i, sz, vp, sz, sz, vp]
        L.oracle_symm_f64.restype = i
        L.oracle_symm_f64.argtypes = [i, i, i, i, i, sz, sz, dp, vp, sz, sz, vp, sz, sz, dp, vp, sz, sz]
        L.oracle_syrk_f64.restype = i
        L.oracle_syrk_f64.argtypes = [i, i, i, i, i, sz, sz, dp, vp, sz, sz, dp, vp, sz, sz]
        L.oracle_syr2k_f64.restype = i
        L.oracle_syr2k_f64.argtypes = [i, i, i, i, i, sz, sz, dp, vp, sz, sz, vp, sz, sz, dp, vp, sz, sz]
        for name in ("oracle_trmm_f64", "oracle_trsm_f64"):
            f = getattr(L, name)
            f.restype = i
            f.argtypes = [i, i, i, i, i, i, sz, sz, dp, vp, sz, sz, vp, sz, sz]
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


# ---- level-3 routines built on GEMM (oracle/level3_oracle.c): fp64 results in a widened copy of the output ----------

def _wide(precision, buf):
    c64 = np.ascontiguousarray(widen(precision, buf))
    return c64, c64.view(np.float64)


def expand_triangle(precision, kind, layout, triangle, unit, k, a, a_off, a_ld):
    """The square matrix (k*k entries in memory order, widened) the reference's convert kernels make from a stored
    triangle. kind 0 symmetric, 1 hermitian, 2 triangular."""
    out = np.zeros(k * k, dtype=np.complex128 if precision > 100 else np.float64)
    st = lib().oracle_expand_triangle(precision, kind, int(layout), int(triangle), int(bool(unit)), k, _vp(a), a_off,
                                      a_ld, _vp(out.view(np.float64)))
    assert st == 0
    return out


def symm_f64(precision, layout, side, triangle, m, n, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld,
             hermitian=False):
    c64, view = _wide(precision, c)
    st = lib().oracle_symm_f64(precision, int(hermitian), int(layout), int(side), int(triangle), m, n, _pair(alpha),
                               _vp(a), a_off, a_ld, _vp(b), b_off, b_ld, _pair(beta), _vp(view), c_off, c_ld)
    assert st == 0
    return c64


def syrk_f64(precision, layout, triangle, trans, n, k, alpha, a, a_off, a_ld, beta, c, c_off, c_ld, hermitian=False):
    c64, view = _wide(precision, c)
    st = lib().oracle_syrk_f64(precision, int(hermitian), int(layout), int(triangle), int(trans), n, k, _pair(alpha),
                               _vp(a), a_off, a_ld, _pair(beta), _vp(view), c_off, c_ld)
    assert st == 0
    return c64


def syr2k_f64(precision, layout, triangle, trans, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld,
              hermitian=False):
    c64, view = _wide(precision, c)
    st = lib().oracle_syr2k_f64(precision, int(hermitian), int(layout), int(triangle), int(trans), n, k, _pair(alpha),
                                _vp(a), a_off, a_ld, _vp(b), b_off, b_ld, _pair(beta), _vp(view), c_off, c_ld)
    assert st == 0
    return c64


def trmm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, a_off, a_ld, b, b_off, b_ld):
    b64, view = _wide(precision, b)
    st = lib().oracle_trmm_f64(precision, int(layout), int(side), int(triangle), int(trans), int(diag), m, n,
                               _pair(alpha), _vp(a), a_off, a_ld, _vp(view), b_off, b_ld)
    assert st == 0
    return b64


def trsm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, a_off, a_ld, b, b_off, b_ld):
    b64, view = _wide(precision, b)
    st = lib().oracle_trsm_f64(precision, int(layout), int(side), int(triangle), int(trans), int(diag), m, n,
                               _pair(alpha), _vp(a), a_off, a_ld, _vp(view), b_off, b_ld)
    assert st == 0
    return b64


# ---- the copies either side of the GEMM path: index arithmetic in numpy ------------------------------------------

def omatcopy(precision, layout, trans, m, n, alpha, a, a_off, a_ld, b, b_off, b_ld):
    """B = alpha * op(A) on host buffers, in the routine's own type (reference: src/routines/levelx/xomatcopy.cpp:45-78;
    host check test/routines/levelx/xomatcopy.hpp:128-150). Returns the updated copy of ``b``."""
    out = b.copy()
    rows, cols = (m, n)
    src = np.empty((rows, cols), dtype=a.dtype)
    for r in range(rows):
        for c in range(cols):
            src[r, c] = a[a_off + (r * a_ld + c if layout == 101 else c * a_ld + r)]
    if trans != 111:
        src = src.T
    if trans == 113:
        src = np.conj(src)
    if precision == 16:
        res = (np.float32(np.float16(alpha)) * src.astype(np.float32)).astype(np.float16)   # alpha arrives as a half
    else:
        res = (NP_OF[precision](alpha) * src).astype(NP_OF[precision])
    for r in range(res.shape[0]):
        for c in range(res.shape[1]):
            out[b_off + (r * b_ld + c if layout == 101 else c * b_ld + r)] = res[r, c]
    return out


def im2col(mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, im, im_off,
           col, col_off):
    """Column matrix of one image (reference: src/kernels/levelx/im2col.opencl:24-62). Returns the updated copy of ``col``."""
    oh, ow = conv_output_size(height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w)
    out = col.copy()
    image = im[im_off:im_off + channels * height * width].reshape(channels, height, width)
    ho, wo = np.arange(oh)[:, None], np.arange(ow)[None, :]
    for c in range(channels):
        for kh in range(kernel_h):
            for kw in range(kernel_w):
                h = ho * stride_h - pad_h + kh * dil_h
                w = wo * stride_w - pad_w + kw * dil_w
                ok = (h >= 0) & (h < height) & (w >= 0) & (w < width)
                vals = np.where(ok, image[c][np.clip(h, 0, height - 1), np.clip(w, 0, width - 1)], 0).astype(im.dtype)
                kidx = kernel_h * kernel_w - kw - kernel_w * kh - 1 if mode == 152 else kw + kernel_w * kh
                base = col_off + (c * kernel_h * kernel_w + kidx) * oh * ow
                out[base:base + oh * ow] = vals.ravel()
    return out


def col2im(mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, col,
           col_off, im, im_off):
    """im += the column entries im2col would have read from each pixel, summed per pixel in the reference's order: taps
    from the last kernel row and column to the first, in the routine's own type (reference:
    src/kernels/levelx/col2im.opencl:29-89). Returns the updated copy of ``im``."""
    oh, ow = conv_output_size(height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w)
    dt = im.dtype
    sums = np.zeros((channels, height, width), dtype=dt)
    touched = np.zeros((channels, height, width), dtype=bool)
    columns = col[col_off:col_off + channels * kernel_h * kernel_w * oh * ow].reshape(channels, kernel_h * kernel_w, oh, ow)
    for kh in range(kernel_h - 1, -1, -1):
        for kw in range(kernel_w - 1, -1, -1):
            kidx = kernel_h * kernel_w - kw - kernel_w * kh - 1 if mode == 152 else kw + kernel_w * kh
            for ho in range(oh):
                h = ho * stride_h - pad_h + kh * dil_h
                if h < 0 or h >= height:
                    continue
                w = np.arange(ow) * stride_w - pad_w + kw * dil_w
                ok = (w >= 0) & (w < width)
                sums[:, h, w[ok]] = (sums[:, h, w[ok]] + columns[:, kidx, ho, ok]).astype(dt)
                touched[:, h, w[ok]] = True
    out = im.copy()
    view = out[im_off:im_off + channels * height * width].reshape(channels, height, width)
    view[touched] = (view[touched] + sums[touched]).astype(dt)
    return out


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
