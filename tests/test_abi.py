"""CPU-side checks of the drop-in boundary: the library loads, exports every declared symbol, and the host
logic that needs no device behaves like the reference's."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

import clblast_b200 as cb
from clblast_b200._lib import C_ABI_SYMBOLS, C_API_SYMBOLS, LIB_PATH, NETLIB_SYMBOLS

ROOT = Path(__file__).resolve().parent.parent


def test_library_loads_and_reports_version():
    assert b"sm_100a" in cb.lib().b200blas_version()


def test_every_declared_c_symbol_is_exported():
    header = (ROOT / "include" / "b200blas.h").read_text()
    declared = set(re.findall(r"\b(b200blas_\w+)\s*\(", header))
    assert declared == set(C_ABI_SYMBOLS)
    L = cb.lib()
    for name in declared:
        assert getattr(L, name) is not None


def test_c_and_netlib_style_layers_export_every_declared_symbol():
    c_header = (ROOT / "include" / "b200blas_c.h").read_text()
    n_header = (ROOT / "include" / "b200blas_netlib.h").read_text()
    assert set(re.findall(r"CLBlastStatusCode (CLBlast\w+)\(", c_header)) == set(C_API_SYMBOLS)
    assert set(re.findall(r"void (cblas_\w+)\(", n_header)) == set(NETLIB_SYMBOLS)
    # the names the reference's C API and Netlib layer give these routines (include/clblast_c.h:885,
    # include/clblast_netlib_c.h:402)
    assert "CLBlastSgemm" in C_API_SYMBOLS and "CLBlastZher2k" in C_API_SYMBOLS and "cblas_sgemm" in NETLIB_SYMBOLS
    L = cb.lib()
    for name in C_API_SYMBOLS + NETLIB_SYMBOLS:
        assert getattr(L, name) is not None, name
    # both headers are plain C
    for header in ("b200blas_c.h", "b200blas_netlib.h"):
        src = f'#include "{header}"\nint main(void) {{ return 0; }}\n'
        res = subprocess.run(["gcc", "-std=c99", "-fsyntax-only", "-x", "c", "-I", str(ROOT / "include"), "-I",
                              "/usr/local/cuda/include", "-"], input=src, capture_output=True, text=True)
        assert res.returncode == 0, res.stderr


def test_level3_cxx_symbols_are_exported():
    out = subprocess.run(["nm", "-D", "--defined-only", str(LIB_PATH)], capture_output=True, text=True, check=True).stdout
    syms = {line.split()[-1] for line in out.splitlines() if line.strip()}
    for routine in ("Symm", "Syrk", "Syr2k", "Trmm", "Omatcopy", "Im2col", "Col2im"):
        for t in ("f", "d", "t", "St7complexIfE", "St7complexIdE"):
            assert any(s.startswith(f"_ZN7clblast{len(routine)}{routine}I{t}E") for s in syms), (routine, t)
    for t in ("f", "d", "St7complexIfE", "St7complexIdE"):
        assert any(s.startswith(f"_ZN7clblast4TrsmI{t}E") for s in syms), t
    for t in ("St7complexIfE", "St7complexIdE"):
        assert any(s.startswith(f"_ZN7clblast4HemmI{t}E") for s in syms), t
    assert any(s.startswith("_ZN7clblast4HerkIfE") for s in syms) and any(s.startswith("_ZN7clblast4HerkIdE") for s in syms)
    assert any(s.startswith("_ZN7clblast5Her2kISt7complexIfEfE") for s in syms)
    assert any(s.startswith("_ZN7clblast5Her2kISt7complexIdEdE") for s in syms)


def test_cxx_api_symbols_have_the_reference_mangling():
    out = subprocess.run(["nm", "-D", "--defined-only", str(LIB_PATH)], capture_output=True, text=True, check=True).stdout
    syms = {line.split()[-1] for line in out.splitlines() if line.strip()}
    # clblast::Gemm<float> as exported by the reference's own CUDA build.
    assert "_ZN7clblast4GemmIfEENS_10StatusCodeENS_6LayoutENS_9TransposeES3_mmmT_ymmymmS4_ymmP8CUctx_stiy" in syms
    for t in ("f", "d", "t", "St7complexIfE", "St7complexIdE"):
        assert any(s.startswith(f"_ZN7clblast4GemmI{t}E") for s in syms), t
        assert any(s.startswith(f"_ZN7clblast11GemmBatchedI{t}E") for s in syms), t
        assert any(s.startswith(f"_ZN7clblast18GemmStridedBatchedI{t}E") for s in syms), t
        assert any(s.startswith(f"_ZN7clblast18GemmTempBufferSizeI{t}E") for s in syms), t
    for t in ("f", "d", "t"):
        assert any(s.startswith(f"_ZN7clblast8ConvgemmI{t}E") for s in syms), t
    for name in ("ClearCache", "FillCache", "RetrieveParameters", "OverrideParameters"):
        assert any(f"clblast{len(name)}{name}" in s or f"{len(name)}{name}E" in s for s in syms), name


def test_library_does_not_need_a_driver_to_load():
    out = subprocess.run(["ldd", str(LIB_PATH)], capture_output=True, text=True, check=True).stdout
    assert "libcuda" not in out and "not found" not in out


def test_zero_dimension_is_rejected_before_anything_else():
    for m, n, k in ((0, 4, 4), (4, 0, 4), (4, 4, 0)):
        assert cb.Gemm(cb.Layout.kColMajor, cb.Transpose.kNo, cb.Transpose.kNo, m, n, k, 1.0, 0, 0, 4, 0, 0, 4, 0.0, 0,
                       0, 4, precision=32) == cb.StatusCode.kInvalidDimension


def test_leading_dimension_checks_come_in_a_b_c_order():
    g = lambda lda, ldb, ldc: cb.Gemm(cb.Layout.kColMajor, cb.Transpose.kNo, cb.Transpose.kNo, 8, 8, 8, 1.0, 0, 0, lda,
                                      0, 0, ldb, 0.0, 0, 0, ldc, precision=32)
    assert g(7, 7, 7) == cb.StatusCode.kInvalidLeadDimA
    # a valid lda with a null A buffer is an invalid matrix A, reported before B's leading dimension
    assert g(8, 7, 7) == cb.StatusCode.kInvalidMatrixA


def test_batched_argument_checks():
    S = cb.StatusCode
    assert cb.GemmStridedBatched(102, 111, 111, 4, 4, 4, 1.0, 0, 0, 4, 16, 0, 0, 4, 16, 0.0, 0, 0, 4, 16, 0,
                                 precision=32) == S.kInvalidBatchCount
    assert cb.GemmStridedBatched(102, 111, 111, 4, 4, 4, 1.0, 0, 0, 4, 16, 0, 0, 4, 16, 0.0, 0, 0, 4, 0, 2,
                                 precision=32) == S.kInvalidDimension
    assert cb.GemmBatched(102, 111, 111, 4, 4, 4, [], 0, [], 4, 0, [], 4, [], 0, [], 4, 0,
                          precision=32) == S.kInvalidBatchCount
    assert cb.GemmBatched(102, 111, 111, 4, 4, 4, [1.0], 0, [0, 0], 4, 0, [0], 4, [0.0], 0, [0], 4, 1,
                          precision=32) == S.kInvalidBatchCount


def test_convgemm_argument_checks():
    S = cb.StatusCode
    conv = lambda **kw: cb.Convgemm(151, kw.get("c", 2), kw.get("h", 8), 8, 3, 3, 1, 1, 1, 1, 1, 1, kw.get("k", 4),
                                    kw.get("b", 2), 0, 0, 0, 0, 0, 0, precision=32)
    assert conv(b=0) == S.kInvalidBatchCount
    assert conv(c=0) == S.kInvalidDimension
    assert conv(h=0) == S.kInvalidDimension
    assert conv(k=0) == S.kInvalidDimension
    assert conv() == S.kInvalidMatrixB  # weights are validated first, the image never
    assert cb.Convgemm(151, 2, 8, 8, 3, 3, 1, 1, 1, 1, 1, 1, 4, 2, 0, 0, 0, 0, 0, 0,
                       precision=3232) == S.kNotImplemented


def test_temp_buffer_size_is_zero():
    st, size = cb.GemmTempBufferSize(102, 111, 112, 4096, 4096, 4096, 0, 4096, 0, 4096, 0, 4096, precision=32)
    assert st == cb.StatusCode.kSuccess and size == 0
    st, _ = cb.GemmTempBufferSize(102, 111, 112, 0, 4096, 4096, 0, 4096, 0, 4096, 0, 4096, precision=32)
    assert st == cb.StatusCode.kInvalidDimension


def test_cache_calls_are_accepted():
    assert cb.ClearCache() == cb.StatusCode.kSuccess
    assert cb.FillCache(0) == cb.StatusCode.kSuccess


XGEMM_NAMES = ["GEMMK", "KREG", "KWG", "KWI", "MDIMA", "MDIMC", "MWG", "NDIMB", "NDIMC", "NWG", "SA", "SB", "STRM",
               "STRN", "VWM", "VWN"]


def test_retrieve_parameters_lists_every_xgemm_name():
    # what the reference's retrieve_parameters test expects: all names present, values below 16384
    for prec in (16, 32, 64, 3232, 6464):
        st, params = cb.RetrieveParameters(0, "Xgemm", prec)
        assert st == cb.StatusCode.kSuccess
        assert set(params) == set(XGEMM_NAMES)
        assert all(v < 16384 for v in params.values())
    for fam in ("XgemmDirect", "GemmRoutine", "Xconvgemm", "Copy", "Pad", "Transpose", "Padtranspose"):
        st, params = cb.RetrieveParameters(0, fam, 32)
        assert st == cb.StatusCode.kSuccess and params
    st, _ = cb.RetrieveParameters(0, "NoSuchKernel", 32)
    assert st == cb.StatusCode.kDatabaseError


def test_override_parameters_needs_the_full_family():
    full = {name: 8 for name in XGEMM_NAMES}
    partial = {name: 8 for name in XGEMM_NAMES[:10]}
    assert cb.OverrideParameters(1, "Xgemm", 32, partial) == cb.StatusCode.kMissingOverrideParameter
    assert cb.OverrideParameters(1, "Xgemm", 32, full) == cb.StatusCode.kSuccess
    assert cb.OverrideParameters(1, "Xgemm", 32, dict(full, EXTRA=1)) == cb.StatusCode.kSuccess
    st, params = cb.RetrieveParameters(1, "Xgemm", 32)
    assert st == cb.StatusCode.kSuccess and all(v == 8 for v in params.values())
    # other devices and precisions keep their own values
    _, other = cb.RetrieveParameters(0, "Xgemm", 32)
    assert other["MWG"] != 8
    assert cb.OverrideParameters(1, "NoSuchKernel", 32, full) == cb.StatusCode.kDatabaseError
