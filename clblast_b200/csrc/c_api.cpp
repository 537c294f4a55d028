// The C interface of include/b200blas_c.h: one forward per routine and element type to the flat C ABI
// (include/b200blas.h), with the given context made current for the duration of the call. Reference counterpart:
// src/clblast_c.cpp (OpenCL flavour only).
#include "b200blas_c.h"

#include "api_shim.h"
#include "b200blas.h"

namespace {
inline const void* P(CUdeviceptr p) { return reinterpret_cast<const void*>(p); }
inline void* PM(CUdeviceptr p) { return reinterpret_cast<void*>(p); }
}  // namespace

#define B200_C_CALL(expr)                        \
  try {                                          \
    clblast::shim::ContextGuard guard(context);  \
    (void)device;                                \
    return (expr);                               \
  } catch (...) {                                \
    return -2039;                                \
  }

extern "C" CLBlastStatusCode CLBlastSgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const float alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm(32, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const double alpha, const
    CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset,
    const size_t b_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm(64, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexFloat alpha,
    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const
    size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm(3232, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexDouble alpha,
    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const
    size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm(6464, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf alpha, const
    CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset,
    const size_t b_ld, const CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm(16, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const float beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_symm(32, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const double alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const double beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_symm(64, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device) {
  B200_C_CALL(b200blas_symm(3232, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_symm(6464, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_symm(16, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastChemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device) {
  B200_C_CALL(b200blas_hemm(3232, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZhemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const size_t m, const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_hemm(6464, layout, side, triangle, m, n, &alpha, P(a_buffer), a_offset, a_ld, P(b_buffer),
    b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t
    c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syrk(32, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const
    size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syrk(64, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CLBlastComplexFloat beta, CUdeviceptr c_buffer, const
    size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syrk(3232, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CLBlastComplexDouble beta, CUdeviceptr c_buffer, const
    size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syrk(6464, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const CLBlastHalf alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset,
    const size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syrk(16, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t
    c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_herk(3232, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const
    size_t c_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_herk(6464, layout, triangle, a_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld, &beta,
    PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld,
    const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_syr2k(32, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld,
    const double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_syr2k(64, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syr2k(3232, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld,
    const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syr2k(6464, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const CLBlastHalf alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_syr2k(16, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_her2k(3232, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const
    CLBlastTranspose ab_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_her2k(6464, layout, triangle, ab_transpose, n, k, &alpha, P(a_buffer), a_offset, a_ld,
    P(b_buffer), b_offset, b_ld, &beta, PM(c_buffer), c_offset, c_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastStrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const float alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trmm(32, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const double alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trmm(64, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trmm(3232, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trmm(6464, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trmm(16, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastStrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const float alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trsm(32, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const double alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trsm(64, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trsm(3232, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle
    triangle, const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n,
    const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_trsm(6464, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, P(a_buffer), a_offset,
    a_ld, PM(b_buffer), b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    size_t m, const size_t n, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_omatcopy(32, layout, a_transpose, m, n, &alpha, P(a_buffer), a_offset, a_ld, PM(b_buffer),
    b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    size_t m, const size_t n, const double alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t
    a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice
    device) {
  B200_C_CALL(b200blas_omatcopy(64, layout, a_transpose, m, n, &alpha, P(a_buffer), a_offset, a_ld, PM(b_buffer),
    b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastComatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    size_t m, const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_omatcopy(3232, layout, a_transpose, m, n, &alpha, P(a_buffer), a_offset, a_ld, PM(b_buffer),
    b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    size_t m, const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_omatcopy(6464, layout, a_transpose, m, n, &alpha, P(a_buffer), a_offset, a_ld, PM(b_buffer),
    b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    size_t m, const size_t n, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t
    a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice
    device) {
  B200_C_CALL(b200blas_omatcopy(16, layout, a_transpose, m, n, &alpha, P(a_buffer), a_offset, a_ld, PM(b_buffer),
    b_offset, b_ld, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_im2col(32, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(im_buffer), im_offset, PM(col_buffer), col_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_im2col(64, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(im_buffer), im_offset, PM(col_buffer), col_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_im2col(3232, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(im_buffer), im_offset, PM(col_buffer), col_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_im2col(6464, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(im_buffer), im_offset, PM(col_buffer), col_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_im2col(16, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(im_buffer), im_offset, PM(col_buffer), col_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastScol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_col2im(32, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(col_buffer), col_offset, PM(im_buffer), im_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_col2im(64, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(col_buffer), col_offset, PM(im_buffer), im_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_col2im(3232, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(col_buffer), col_offset, PM(im_buffer), im_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_col2im(6464, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(col_buffer), col_offset, PM(im_buffer), im_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device) {
  B200_C_CALL(b200blas_col2im(16, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, P(col_buffer), col_offset, PM(im_buffer), im_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_convgemm(32, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, num_kernels, batch_count, P(im_buffer), im_offset, P(kernel_buffer),
    kernel_offset, PM(result_buffer), result_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_convgemm(64, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, num_kernels, batch_count, P(im_buffer), im_offset, P(kernel_buffer),
    kernel_offset, PM(result_buffer), result_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t
    height, const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device) {
  B200_C_CALL(b200blas_convgemm(16, kernel_mode, channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h,
    stride_w, dilation_h, dilation_w, num_kernels, batch_count, P(im_buffer), im_offset, P(kernel_buffer),
    kernel_offset, PM(result_buffer), result_offset, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const float* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const float* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const size_t
    c_ld, const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_batched(32, layout, a_transpose, b_transpose, m, n, k, alphas, P(a_buffer), a_offsets,
    a_ld, P(b_buffer), b_offsets, b_ld, betas, PM(c_buffer), c_offsets, c_ld, batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const double* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const double* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const size_t
    c_ld, const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_batched(64, layout, a_transpose, b_transpose, m, n, k, alphas, P(a_buffer), a_offsets,
    a_ld, P(b_buffer), b_offsets, b_ld, betas, PM(c_buffer), c_offsets, c_ld, batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexFloat* alphas,
    const CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastComplexFloat* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
    const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_batched(3232, layout, a_transpose, b_transpose, m, n, k, alphas, P(a_buffer), a_offsets,
    a_ld, P(b_buffer), b_offsets, b_ld, betas, PM(c_buffer), c_offsets, c_ld, batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexDouble* alphas,
    const CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastComplexDouble* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
    const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_batched(6464, layout, a_transpose, b_transpose, m, n, k, alphas, P(a_buffer), a_offsets,
    a_ld, P(b_buffer), b_offsets, b_ld, betas, PM(c_buffer), c_offsets, c_ld, batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastHalf* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const
    size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_batched(16, layout, a_transpose, b_transpose, m, n, k, alphas, P(a_buffer), a_offsets,
    a_ld, P(b_buffer), b_offsets, b_ld, betas, PM(c_buffer), c_offsets, c_ld, batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastSgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose
    a_transpose, const CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const float
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const float beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count,
    const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_strided_batched(32, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer),
    a_offset, a_ld, a_stride, P(b_buffer), b_offset, b_ld, b_stride, &beta, PM(c_buffer), c_offset, c_ld, c_stride,
    batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastDgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose
    a_transpose, const CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const double
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const double beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count,
    const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_strided_batched(64, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer),
    a_offset, a_ld, a_stride, P(b_buffer), b_offset, b_ld, b_stride, &beta, PM(c_buffer), c_offset, c_ld, c_stride,
    batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastCgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose
    a_transpose, const CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const
    CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t
    a_stride, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride,
    const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_strided_batched(3232, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer),
    a_offset, a_ld, a_stride, P(b_buffer), b_offset, b_ld, b_stride, &beta, PM(c_buffer), c_offset, c_ld, c_stride,
    batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastZgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose
    a_transpose, const CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const
    CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t
    a_stride, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride,
    const size_t batch_count, const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_strided_batched(6464, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer),
    a_offset, a_ld, a_stride, P(b_buffer), b_offset, b_ld, b_stride, &beta, PM(c_buffer), c_offset, c_ld, c_stride,
    batch_count, 0, 0))
}
extern "C" CLBlastStatusCode CLBlastHgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose
    a_transpose, const CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const CLBlastHalf beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count,
    const CUcontext context, const CUdevice device) {
  B200_C_CALL(b200blas_gemm_strided_batched(16, layout, a_transpose, b_transpose, m, n, k, &alpha, P(a_buffer),
    a_offset, a_ld, a_stride, P(b_buffer), b_offset, b_ld, b_stride, &beta, PM(c_buffer), c_offset, c_ld, c_stride,
    batch_count, 0, 0))
}
