"""ctypes front end of oracle/_ref/libclblast_ref_kernels.so (the reference's kernel source run on the CPU).

TEST INFRASTRUCTURE ONLY: used by tests/test_oracle_ref.py to pin the C oracle to the reference's arithmetic."""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p

import numpy as np

from . import build_ref

TAGS = build_ref.PRECISIONS
NP_OF = {16: np.float16, 32: np.float32, 64: np.float64, 3232: np.complex64, 6464: np.complex128}
_lib = None


def available() -> bool:
    return build_ref.LIB_PATH.exists() or build_ref.reference_available()


def lib():
    global _lib
    if _lib is None:
        if not build_ref.LIB_PATH.exists():
            build_ref.build()
        L = ctypes.CDLL(str(build_ref.LIB_PATH))
        for tag in TAGS.values():
            f = getattr(L, f"ref_gemm_direct_{tag}")
            f.restype = c_int
            f.argtypes = [c_int] * 6 + [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                        c_int, c_int]
        for tag in ("p16", "p32", "p64"):
            f = getattr(L, f"ref_convgemm_{tag}")
            f.restype = c_int
            f.argtypes = [c_int] * 14 + [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int]
        for tag in TAGS.values():
            f = getattr(L, f"ref_expand_triangle_{tag}")
            f.restype = c_int
            f.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p]
            for name in ("ref_im2col", "ref_col2im"):
                f = getattr(L, f"{name}_{tag}")
                f.restype = c_int
                f.argtypes = [c_int] * 12 + [c_void_p, c_int, c_void_p, c_int]
        _lib = L
    return _lib


def _vp(a):
    return a.ctypes.data_as(c_void_p)


def gemm_direct(precision, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld):
    """Runs the reference's XgemmDirect{NN,NT,TN,TT} kernel on host buffers, in place on ``c``."""
    dt = NP_OF[precision]
    al, be = np.array([alpha], dtype=dt), np.array([beta], dtype=dt)
    fn = getattr(lib(), f"ref_gemm_direct_{TAGS[precision]}")
    st = fn(int(layout), int(ta), int(tb), m, n, k, _vp(al), _vp(a), a_off, a_ld, _vp(b), b_off, b_ld, _vp(be), _vp(c),
            c_off, c_ld)
    assert st == 0
    return c


def convgemm(precision, mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h,
             dil_w, num_kernels, batch_count, im, im_off, ker, ker_off, result, result_off):
    """Runs the reference's XconvgemmNormal / XconvgemmFlip kernel on host buffers, in place on ``result``."""
    fn = getattr(lib(), f"ref_convgemm_{TAGS[precision]}")
    st = fn(int(mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
            num_kernels, batch_count, _vp(im), im_off, _vp(ker), ker_off, _vp(result), result_off)
    assert st == 0
    return result


def expand_triangle(precision, kind, layout, triangle, unit, k, a, a_off, a_ld):
    """Runs the reference's {Symm,Herm,Tria}{Upper,Lower}ToSquared kernel (kind 0, 1, 2) the way Xsymm / Xhemm / Xtrmm
    choose and launch it; returns the k*k result in the routine's own type."""
    upper = (triangle == 121) != (layout == 101)
    out = np.zeros(k * k, dtype=NP_OF[precision])
    fn = getattr(lib(), f"ref_expand_triangle_{TAGS[precision]}")
    assert fn(kind, int(upper), int(bool(unit)), k, _vp(a), a_off, a_ld, _vp(out)) == 0
    return out


def im2col(precision, mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
           im, im_off, col, col_off):
    """Runs the reference's Xim2colKernelNormal / Flip on host buffers, in place on ``col``."""
    fn = getattr(lib(), f"ref_im2col_{TAGS[precision]}")
    assert fn(int(mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
              _vp(im), im_off, _vp(col), col_off) == 0
    return col


def col2im(precision, mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
           col, col_off, im, im_off):
    """Runs the reference's Xcol2imKernelNormal / Flip on host buffers, in place on ``im``."""
    fn = getattr(lib(), f"ref_col2im_{TAGS[precision]}")
    assert fn(int(mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
              _vp(col), col_off, _vp(im), im_off) == 0
    return im
