// Stand-in for the reference's test/wrapper_cblas.hpp, used only when the reference's own test programs are
// built against this library (tests/ref_harness/build.py). The original wraps ~100 CBLAS routines and needs
// <cblas.h>; the tests of the GEMM family and of the level-3 routines built on it only use convertToCBLAS and the
// cblasXgemm / Xsymm / Xhemm / Xsyrk / Xherk / Xsyr2k / Xher2k / Xtrmm / Xtrsm overloads, which are provided here on
// top of this repository's CPU oracle (fp64 arithmetic, rounded once to the routine's type).
#ifndef CLBLAST_TEST_WRAPPER_CBLAS_H_
#define CLBLAST_TEST_WRAPPER_CBLAS_H_

#include <complex>
#include <cstddef>
#include <vector>

#include "clblast.h"
#include "clblast_half.h"
#include "test/test_utilities.hpp"
#include "utilities/utilities.hpp"

extern "C" int oracle_gemm_f64(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k,
                               const double* alpha, const void* a, size_t a_off, size_t a_ld, const void* b,
                               size_t b_off, size_t b_ld, const double* beta, double* c64, size_t c_off, size_t c_ld);

extern "C" {
int oracle_symm_f64(int dtype, int hermitian, int layout, int side, int triangle, size_t m, size_t n, const double* alpha,
                    const void* a, size_t a_off, size_t a_ld, const void* b, size_t b_off, size_t b_ld,
                    const double* beta, double* c64, size_t c_off, size_t c_ld);
int oracle_syrk_f64(int dtype, int hermitian, int layout, int triangle, int trans, size_t n, size_t k, const double* alpha,
                    const void* a, size_t a_off, size_t a_ld, const double* beta, double* c64, size_t c_off, size_t c_ld);
int oracle_syr2k_f64(int dtype, int hermitian, int layout, int triangle, int trans, size_t n, size_t k,
                     const double* alpha, const void* a, size_t a_off, size_t a_ld, const void* b, size_t b_off,
                     size_t b_ld, const double* beta, double* c64, size_t c_off, size_t c_ld);
int oracle_trmm_f64(int dtype, int layout, int side, int triangle, int trans, int diag, size_t m, size_t n,
                    const double* alpha, const void* a, size_t a_off, size_t a_ld, double* b64, size_t b_off, size_t b_ld);
int oracle_trsm_f64(int dtype, int layout, int side, int triangle, int trans, int diag, size_t m, size_t n,
                    const double* alpha, const void* a, size_t a_off, size_t a_ld, double* b64, size_t b_off, size_t b_ld);
}

namespace clblast {

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
enum CBLAS_UPLO { CblasUpper = 121, CblasLower = 122 };
enum CBLAS_DIAG { CblasNonUnit = 131, CblasUnit = 132 };
enum CBLAS_SIDE { CblasLeft = 141, CblasRight = 142 };

inline CBLAS_ORDER convertToCBLAS(const Layout v) { return (v == Layout::kRowMajor) ? CblasRowMajor : CblasColMajor; }
inline CBLAS_TRANSPOSE convertToCBLAS(const Transpose v) {
  return (v == Transpose::kNo) ? CblasNoTrans : (v == Transpose::kYes) ? CblasTrans : CblasConjTrans;
}
inline CBLAS_UPLO convertToCBLAS(const Triangle v) { return (v == Triangle::kUpper) ? CblasUpper : CblasLower; }
inline CBLAS_DIAG convertToCBLAS(const Diagonal v) { return (v == Diagonal::kUnit) ? CblasUnit : CblasNonUnit; }
inline CBLAS_SIDE convertToCBLAS(const Side v) { return (v == Side::kLeft) ? CblasLeft : CblasRight; }

namespace oracle_detail {

template <typename T> struct Info;
template <> struct Info<float> { static constexpr int dtype = 32; static constexpr int parts = 1; using R = float; };
template <> struct Info<double> { static constexpr int dtype = 64; static constexpr int parts = 1; using R = double; };
template <> struct Info<std::complex<float>> { static constexpr int dtype = 3232; static constexpr int parts = 2; using R = float; };
template <> struct Info<std::complex<double>> { static constexpr int dtype = 6464; static constexpr int parts = 2; using R = double; };

template <typename T>
void gemm(int layout, int ta, int tb, size_t m, size_t n, size_t k, const T alpha, const std::vector<T>& a,
          size_t a_offset, size_t a_ld, const std::vector<T>& b, size_t b_offset, size_t b_ld, const T beta,
          std::vector<T>& c, size_t c_offset, size_t c_ld) {
  using R = typename Info<T>::R;
  constexpr int parts = Info<T>::parts;
  const std::complex<double> al(alpha), be(beta);
  const double alpha2[2] = {al.real(), al.imag()}, beta2[2] = {be.real(), be.imag()};
  std::vector<double> wide(c.size() * parts);
  const R* c_raw = reinterpret_cast<const R*>(c.data());
  for (size_t i = 0; i < wide.size(); ++i) wide[i] = static_cast<double>(c_raw[i]);
  oracle_gemm_f64(Info<T>::dtype, layout, ta, tb, m, n, k, alpha2, a.data(), a_offset, a_ld, b.data(), b_offset, b_ld,
                  beta2, wide.data(), c_offset, c_ld);
  R* c_out = reinterpret_cast<R*>(c.data());
  for (size_t i = 0; i < wide.size(); ++i) c_out[i] = static_cast<R>(wide[i]);
}

}  // namespace oracle_detail

#define B200_CBLAS_GEMM(T)                                                                                          \
  inline void cblasXgemm(const CBLAS_ORDER layout, const CBLAS_TRANSPOSE a_transpose,                              \
                         const CBLAS_TRANSPOSE b_transpose, const size_t m, const size_t n, const size_t k,         \
                         const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,   \
                         const std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld, const T beta,    \
                         std::vector<T>& c_buffer, const size_t c_offset, const size_t c_ld) {                      \
    oracle_detail::gemm<T>(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld, b_buffer,    \
                           b_offset, b_ld, beta, c_buffer, c_offset, c_ld);                                         \
  }
B200_CBLAS_GEMM(float)
B200_CBLAS_GEMM(double)
B200_CBLAS_GEMM(float2)
B200_CBLAS_GEMM(double2)
#undef B200_CBLAS_GEMM

// Half goes through single precision and back, as the reference's wrapper does.
inline void cblasXgemm(const CBLAS_ORDER layout, const CBLAS_TRANSPOSE a_transpose, const CBLAS_TRANSPOSE b_transpose,
                       const size_t m, const size_t n, const size_t k, const half alpha,
                       const std::vector<half>& a_buffer, const size_t a_offset, const size_t a_ld,
                       const std::vector<half>& b_buffer, const size_t b_offset, const size_t b_ld, const half beta,
                       std::vector<half>& c_buffer, const size_t c_offset, const size_t c_ld) {
  auto a_float = HalfToFloatBuffer(a_buffer);
  auto b_float = HalfToFloatBuffer(b_buffer);
  auto c_float = HalfToFloatBuffer(c_buffer);
  cblasXgemm(layout, a_transpose, b_transpose, m, n, k, HalfToFloat(alpha), a_float, a_offset, a_ld, b_float,
             b_offset, b_ld, HalfToFloat(beta), c_float, c_offset, c_ld);
  FloatToHalfBuffer(c_buffer, c_float);
}

// ---- level-3 routines built on GEMM ---------------------------------------------------------------------------------

namespace oracle_detail {

template <> struct Info<half> { static constexpr int dtype = 16; static constexpr int parts = 1; using R = half; };

template <typename T> inline void scalar_pair(const T v, double out[2]) {
  const std::complex<double> z(v);
  out[0] = z.real();
  out[1] = z.imag();
}
template <> inline void scalar_pair<half>(const half v, double out[2]) {
  out[0] = HalfToFloat(v);
  out[1] = 0.0;
}

// The written matrix widened to double (pairs for the complex types), and back.
template <typename T> inline std::vector<double> widen(const std::vector<T>& x) {
  constexpr int parts = Info<T>::parts;
  std::vector<double> w(x.size() * parts);
  const typename Info<T>::R* raw = reinterpret_cast<const typename Info<T>::R*>(x.data());
  for (size_t i = 0; i < w.size(); ++i) w[i] = static_cast<double>(raw[i]);
  return w;
}
template <> inline std::vector<double> widen<half>(const std::vector<half>& x) {
  std::vector<double> w(x.size());
  for (size_t i = 0; i < w.size(); ++i) w[i] = HalfToFloat(x[i]);
  return w;
}
template <typename T> inline void narrow(std::vector<T>& x, const std::vector<double>& w) {
  typename Info<T>::R* raw = reinterpret_cast<typename Info<T>::R*>(x.data());
  for (size_t i = 0; i < w.size(); ++i) raw[i] = static_cast<typename Info<T>::R>(w[i]);
}
template <> inline void narrow<half>(std::vector<half>& x, const std::vector<double>& w) {
  for (size_t i = 0; i < w.size(); ++i) x[i] = FloatToHalf(static_cast<float>(w[i]));
}

}  // namespace oracle_detail

template <typename T>
void cblasXsymm(const CBLAS_ORDER layout, const CBLAS_SIDE side, const CBLAS_UPLO triangle, const size_t m, const size_t n,
                const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                const std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                std::vector<T>& c_buffer, const size_t c_offset, const size_t c_ld) {
  double al[2], be[2];
  oracle_detail::scalar_pair(alpha, al);
  oracle_detail::scalar_pair(beta, be);
  auto wide = oracle_detail::widen(c_buffer);
  oracle_symm_f64(oracle_detail::Info<T>::dtype, 0, layout, side, triangle, m, n, al, a_buffer.data(), a_offset, a_ld,
                  b_buffer.data(), b_offset, b_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename T>
void cblasXhemm(const CBLAS_ORDER layout, const CBLAS_SIDE side, const CBLAS_UPLO triangle, const size_t m, const size_t n,
                const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                const std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                std::vector<T>& c_buffer, const size_t c_offset, const size_t c_ld) {
  double al[2], be[2];
  oracle_detail::scalar_pair(alpha, al);
  oracle_detail::scalar_pair(beta, be);
  auto wide = oracle_detail::widen(c_buffer);
  oracle_symm_f64(oracle_detail::Info<T>::dtype, 1, layout, side, triangle, m, n, al, a_buffer.data(), a_offset, a_ld,
                  b_buffer.data(), b_offset, b_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename T>
void cblasXsyrk(const CBLAS_ORDER layout, const CBLAS_UPLO triangle, const CBLAS_TRANSPOSE a_transpose, const size_t n,
                const size_t k, const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                const T beta, std::vector<T>& c_buffer, const size_t c_offset, const size_t c_ld) {
  double al[2], be[2];
  oracle_detail::scalar_pair(alpha, al);
  oracle_detail::scalar_pair(beta, be);
  auto wide = oracle_detail::widen(c_buffer);
  oracle_syrk_f64(oracle_detail::Info<T>::dtype, 0, layout, triangle, a_transpose, n, k, al, a_buffer.data(), a_offset,
                  a_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename U>
void cblasXherk(const CBLAS_ORDER layout, const CBLAS_UPLO triangle, const CBLAS_TRANSPOSE a_transpose, const size_t n,
                const size_t k, const U alpha, const std::vector<std::complex<U>>& a_buffer, const size_t a_offset,
                const size_t a_ld, const U beta, std::vector<std::complex<U>>& c_buffer, const size_t c_offset,
                const size_t c_ld) {
  using T = std::complex<U>;
  const double al[2] = {static_cast<double>(alpha), 0.0}, be[2] = {static_cast<double>(beta), 0.0};
  auto wide = oracle_detail::widen(c_buffer);
  oracle_syrk_f64(oracle_detail::Info<T>::dtype, 1, layout, triangle, a_transpose, n, k, al, a_buffer.data(), a_offset,
                  a_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename T>
void cblasXsyr2k(const CBLAS_ORDER layout, const CBLAS_UPLO triangle, const CBLAS_TRANSPOSE ab_transpose, const size_t n,
                 const size_t k, const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                 const std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                 std::vector<T>& c_buffer, const size_t c_offset, const size_t c_ld) {
  double al[2], be[2];
  oracle_detail::scalar_pair(alpha, al);
  oracle_detail::scalar_pair(beta, be);
  auto wide = oracle_detail::widen(c_buffer);
  oracle_syr2k_f64(oracle_detail::Info<T>::dtype, 0, layout, triangle, ab_transpose, n, k, al, a_buffer.data(), a_offset,
                   a_ld, b_buffer.data(), b_offset, b_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename U>
void cblasXher2k(const CBLAS_ORDER layout, const CBLAS_UPLO triangle, const CBLAS_TRANSPOSE ab_transpose, const size_t n,
                 const size_t k, const std::complex<U> alpha, const std::vector<std::complex<U>>& a_buffer,
                 const size_t a_offset, const size_t a_ld, const std::vector<std::complex<U>>& b_buffer,
                 const size_t b_offset, const size_t b_ld, const U beta, std::vector<std::complex<U>>& c_buffer,
                 const size_t c_offset, const size_t c_ld) {
  using T = std::complex<U>;
  double al[2];
  oracle_detail::scalar_pair(alpha, al);
  const double be[2] = {static_cast<double>(beta), 0.0};
  auto wide = oracle_detail::widen(c_buffer);
  oracle_syr2k_f64(oracle_detail::Info<T>::dtype, 1, layout, triangle, ab_transpose, n, k, al, a_buffer.data(), a_offset,
                   a_ld, b_buffer.data(), b_offset, b_ld, be, wide.data(), c_offset, c_ld);
  oracle_detail::narrow(c_buffer, wide);
}

template <typename T>
void cblasXtrmm(const CBLAS_ORDER layout, const CBLAS_SIDE side, const CBLAS_UPLO triangle,
                const CBLAS_TRANSPOSE a_transpose, const CBLAS_DIAG diagonal, const size_t m, const size_t n,
                const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld) {
  double al[2];
  oracle_detail::scalar_pair(alpha, al);
  auto wide = oracle_detail::widen(b_buffer);
  oracle_trmm_f64(oracle_detail::Info<T>::dtype, layout, side, triangle, a_transpose, diagonal, m, n, al, a_buffer.data(),
                  a_offset, a_ld, wide.data(), b_offset, b_ld);
  oracle_detail::narrow(b_buffer, wide);
}

template <typename T>
void cblasXtrsm(const CBLAS_ORDER layout, const CBLAS_SIDE side, const CBLAS_UPLO triangle,
                const CBLAS_TRANSPOSE a_transpose, const CBLAS_DIAG diagonal, const size_t m, const size_t n,
                const T alpha, const std::vector<T>& a_buffer, const size_t a_offset, const size_t a_ld,
                std::vector<T>& b_buffer, const size_t b_offset, const size_t b_ld) {
  double al[2];
  oracle_detail::scalar_pair(alpha, al);
  auto wide = oracle_detail::widen(b_buffer);
  oracle_trsm_f64(oracle_detail::Info<T>::dtype, layout, side, triangle, a_transpose, diagonal, m, n, al, a_buffer.data(),
                  a_offset, a_ld, wide.data(), b_offset, b_ld);
  oracle_detail::narrow(b_buffer, wide);
}

}  // namespace clblast

#endif  // CLBLAST_TEST_WRAPPER_CBLAS_H_
