// Stand-in for the reference's test/wrapper_cblas.hpp, used only when the reference's own test programs are
// built against this library (tests/ref_harness/build.py). The original wraps ~100 CBLAS routines and needs
// <cblas.h>; the GEMM-family tests only use convertToCBLAS and the five cblasXgemm overloads, which are provided
// here on top of this repository's CPU oracle (fp64 product, rounded once to the routine's type).
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

namespace clblast {

enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };

inline CBLAS_ORDER convertToCBLAS(const Layout v) { return (v == Layout::kRowMajor) ? CblasRowMajor : CblasColMajor; }
inline CBLAS_TRANSPOSE convertToCBLAS(const Transpose v) {
  return (v == Transpose::kNo) ? CblasNoTrans : (v == Transpose::kYes) ? CblasTrans : CblasConjTrans;
}

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

}  // namespace clblast

#endif  // CLBLAST_TEST_WRAPPER_CBLAS_H_
