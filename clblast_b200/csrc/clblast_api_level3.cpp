// C++ entry points of the level-3 routines that sit on the GEMM path and of the copy / im2col routines either side of
// it, with the reference's names and signatures (include/clblast_cuda.h:393-483; reference definitions and explicit
// instantiations: src/clblast_cuda.cpp:1199-1471, 1510-1623). Thin shims over the C ABI.
#include "clblast_cuda.h"

#include <complex>

#include "api_shim.h"
#include "b200blas.h"

namespace clblast {

#define B200_TRY(expr)                       \
  try {                                      \
    ContextGuard guard(context);             \
    return static_cast<StatusCode>(expr);    \
  } catch (...) {                            \
    return StatusCode::kUnexpectedError;     \
  }

template <typename T>
StatusCode Symm(const Layout layout, const Side side, const Triangle triangle, const size_t m, const size_t n,
                const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice) {
  B200_TRY(b200blas_symm(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(side),
                         static_cast<int>(triangle), m, n, &alpha, dptr(a_buffer), a_offset, a_ld, dptr(b_buffer),
                         b_offset, b_ld, &beta, dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

template <typename T>
StatusCode Hemm(const Layout layout, const Side side, const Triangle triangle, const size_t m, const size_t n,
                const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice) {
  B200_TRY(b200blas_hemm(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(side),
                         static_cast<int>(triangle), m, n, &alpha, dptr(a_buffer), a_offset, a_ld, dptr(b_buffer),
                         b_offset, b_ld, &beta, dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

template <typename T>
StatusCode Syrk(const Layout layout, const Triangle triangle, const Transpose a_transpose, const size_t n,
                const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const T beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice) {
  B200_TRY(b200blas_syrk(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(triangle),
                         static_cast<int>(a_transpose), n, k, &alpha, dptr(a_buffer), a_offset, a_ld, &beta,
                         dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

// T is the real type of alpha and beta; the matrices hold std::complex<T>.
template <typename T>
StatusCode Herk(const Layout layout, const Triangle triangle, const Transpose a_transpose, const size_t n,
                const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const T beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice) {
  B200_TRY(b200blas_herk(DtypeOf<std::complex<T>>::value, static_cast<int>(layout), static_cast<int>(triangle),
                         static_cast<int>(a_transpose), n, k, &alpha, dptr(a_buffer), a_offset, a_ld, &beta,
                         dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

template <typename T>
StatusCode Syr2k(const Layout layout, const Triangle triangle, const Transpose ab_transpose, const size_t n,
                 const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                 const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                 CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                 const CUdevice) {
  B200_TRY(b200blas_syr2k(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(triangle),
                          static_cast<int>(ab_transpose), n, k, &alpha, dptr(a_buffer), a_offset, a_ld, dptr(b_buffer),
                          b_offset, b_ld, &beta, dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

template <typename T, typename U>
StatusCode Her2k(const Layout layout, const Triangle triangle, const Transpose ab_transpose, const size_t n,
                 const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                 const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const U beta,
                 CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                 const CUdevice) {
  B200_TRY(b200blas_her2k(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(triangle),
                          static_cast<int>(ab_transpose), n, k, &alpha, dptr(a_buffer), a_offset, a_ld, dptr(b_buffer),
                          b_offset, b_ld, &beta, dptr_mut(c_buffer), c_offset, c_ld, nullptr, 0))
}

template <typename T>
StatusCode Trmm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose,
                const Diagonal diagonal, const size_t m, const size_t n, const T alpha, const CUdeviceptr a_buffer,
                const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset,
                const size_t b_ld, const CUcontext context, const CUdevice) {
  B200_TRY(b200blas_trmm(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(side),
                         static_cast<int>(triangle), static_cast<int>(a_transpose), static_cast<int>(diagonal), m, n,
                         &alpha, dptr(a_buffer), a_offset, a_ld, dptr_mut(b_buffer), b_offset, b_ld, nullptr, 0))
}

template <typename T>
StatusCode Trsm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose,
                const Diagonal diagonal, const size_t m, const size_t n, const T alpha, const CUdeviceptr a_buffer,
                const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset,
                const size_t b_ld, const CUcontext context, const CUdevice) {
  B200_TRY(b200blas_trsm(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(side),
                         static_cast<int>(triangle), static_cast<int>(a_transpose), static_cast<int>(diagonal), m, n,
                         &alpha, dptr(a_buffer), a_offset, a_ld, dptr_mut(b_buffer), b_offset, b_ld, nullptr, 0))
}

template <typename T>
StatusCode Omatcopy(const Layout layout, const Transpose a_transpose, const size_t m, const size_t n, const T alpha,
                    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
                    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice) {
  B200_TRY(b200blas_omatcopy(DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose), m, n, &alpha,
                             dptr(a_buffer), a_offset, a_ld, dptr_mut(b_buffer), b_offset, b_ld, nullptr, 0))
}

template <typename T>
StatusCode Im2col(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                  const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                  const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                  const CUdeviceptr im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset,
                  const CUcontext context, const CUdevice) {
  B200_TRY(b200blas_im2col(DtypeOf<T>::value, static_cast<int>(kernel_mode), channels, height, width, kernel_h,
                           kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w, dptr(im_buffer),
                           im_offset, dptr_mut(col_buffer), col_offset, nullptr, 0))
}

template <typename T>
StatusCode Col2im(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                  const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                  const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                  const CUdeviceptr col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset,
                  const CUcontext context, const CUdevice) {
  B200_TRY(b200blas_col2im(DtypeOf<T>::value, static_cast<int>(kernel_mode), channels, height, width, kernel_h,
                           kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w, dptr(col_buffer),
                           col_offset, dptr_mut(im_buffer), im_offset, nullptr, 0))
}

// ---- exported instantiations (the same sets as the reference) --------------------------------------------------------

#define B200_ARGS_SYMM(T)                                                                                              \
  (const Layout, const Side, const Triangle, const size_t, const size_t, const T, const CUdeviceptr, const size_t,   \
   const size_t, const CUdeviceptr, const size_t, const size_t, const T, CUdeviceptr, const size_t, const size_t,     \
   const CUcontext, const CUdevice)
#define B200_ARGS_SYRK(T)                                                                                              \
  (const Layout, const Triangle, const Transpose, const size_t, const size_t, const T, const CUdeviceptr,            \
   const size_t, const size_t, const T, CUdeviceptr, const size_t, const size_t, const CUcontext, const CUdevice)
#define B200_ARGS_SYR2K(T, U)                                                                                          \
  (const Layout, const Triangle, const Transpose, const size_t, const size_t, const T, const CUdeviceptr,            \
   const size_t, const size_t, const CUdeviceptr, const size_t, const size_t, const U, CUdeviceptr, const size_t,     \
   const size_t, const CUcontext, const CUdevice)
#define B200_ARGS_TRMM(T)                                                                                              \
  (const Layout, const Side, const Triangle, const Transpose, const Diagonal, const size_t, const size_t, const T,   \
   const CUdeviceptr, const size_t, const size_t, CUdeviceptr, const size_t, const size_t, const CUcontext,           \
   const CUdevice)
#define B200_ARGS_OMATCOPY(T)                                                                                          \
  (const Layout, const Transpose, const size_t, const size_t, const T, const CUdeviceptr, const size_t,              \
   const size_t, CUdeviceptr, const size_t, const size_t, const CUcontext, const CUdevice)
#define B200_ARGS_IM2COL                                                                                               \
  (const KernelMode, const size_t, const size_t, const size_t, const size_t, const size_t, const size_t,             \
   const size_t, const size_t, const size_t, const size_t, const size_t, const CUdeviceptr, const size_t,             \
   CUdeviceptr, const size_t, const CUcontext, const CUdevice)

#define B200_INSTANTIATE_ALL_TYPES(T)                                 \
  template StatusCode PUBLIC_API Symm<T> B200_ARGS_SYMM(T);           \
  template StatusCode PUBLIC_API Syrk<T> B200_ARGS_SYRK(T);           \
  template StatusCode PUBLIC_API Syr2k<T> B200_ARGS_SYR2K(T, T);      \
  template StatusCode PUBLIC_API Trmm<T> B200_ARGS_TRMM(T);           \
  template StatusCode PUBLIC_API Omatcopy<T> B200_ARGS_OMATCOPY(T);   \
  template StatusCode PUBLIC_API Im2col<T> B200_ARGS_IM2COL;          \
  template StatusCode PUBLIC_API Col2im<T> B200_ARGS_IM2COL;

B200_INSTANTIATE_ALL_TYPES(float)
B200_INSTANTIATE_ALL_TYPES(double)
B200_INSTANTIATE_ALL_TYPES(std::complex<float>)
B200_INSTANTIATE_ALL_TYPES(std::complex<double>)
B200_INSTANTIATE_ALL_TYPES(unsigned short)

template StatusCode PUBLIC_API Trsm<float> B200_ARGS_TRMM(float);
template StatusCode PUBLIC_API Trsm<double> B200_ARGS_TRMM(double);
template StatusCode PUBLIC_API Trsm<std::complex<float>> B200_ARGS_TRMM(std::complex<float>);
template StatusCode PUBLIC_API Trsm<std::complex<double>> B200_ARGS_TRMM(std::complex<double>);

template StatusCode PUBLIC_API Hemm<std::complex<float>> B200_ARGS_SYMM(std::complex<float>);
template StatusCode PUBLIC_API Hemm<std::complex<double>> B200_ARGS_SYMM(std::complex<double>);
template StatusCode PUBLIC_API Herk<float> B200_ARGS_SYRK(float);
template StatusCode PUBLIC_API Herk<double> B200_ARGS_SYRK(double);
template StatusCode PUBLIC_API Her2k<std::complex<float>, float> B200_ARGS_SYR2K(std::complex<float>, float);
template StatusCode PUBLIC_API Her2k<std::complex<double>, double> B200_ARGS_SYR2K(std::complex<double>, double);

}  // namespace clblast
