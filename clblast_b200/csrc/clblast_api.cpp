// C++ entry points with the reference's names and signatures (include/clblast_cuda.h), as thin shims over
// the C ABI. The explicit instantiations below are the exported, Itanium-mangled symbols a program built
// against the reference's header resolves at link time (reference: src/clblast_cuda.cpp:1158-1198,
// 1625-1660, 1704-1863; src/api_common.cpp:25-221).
#include "clblast_cuda.h"

#include <complex>
#include <vector>

#include "b200blas.h"

#include "api_shim.h"

namespace clblast {

template <typename T>
StatusCode Gemm(const Layout layout, const Transpose a_transpose, const Transpose b_transpose, const size_t m,
                const size_t n, const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset,
                const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice, CUdeviceptr) {
  try {
    ContextGuard guard(context);
    return static_cast<StatusCode>(b200blas_gemm(
        DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose), static_cast<int>(b_transpose), m,
        n, k, &alpha, dptr(a_buffer), a_offset, a_ld, dptr(b_buffer), b_offset, b_ld, &beta, dptr_mut(c_buffer),
        c_offset, c_ld, nullptr, 0));
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

template <typename T>
StatusCode Convgemm(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                    const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                    const size_t num_kernels, const size_t batch_count, const CUdeviceptr im_buffer,
                    const size_t im_offset, const CUdeviceptr kernel_buffer, const size_t kernel_offset,
                    CUdeviceptr result_buffer, const size_t result_offset, const CUcontext context, const CUdevice) {
  try {
    ContextGuard guard(context);
    return static_cast<StatusCode>(b200blas_convgemm(
        DtypeOf<T>::value, static_cast<int>(kernel_mode), channels, height, width, kernel_h, kernel_w, pad_h, pad_w,
        stride_h, stride_w, dilation_h, dilation_w, num_kernels, batch_count, dptr(im_buffer), im_offset,
        dptr(kernel_buffer), kernel_offset, dptr_mut(result_buffer), result_offset, nullptr, 0));
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

template <typename T>
StatusCode GemmBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose, const size_t m,
                       const size_t n, const size_t k, const T* alphas, const CUdeviceptr a_buffer,
                       const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t* b_offsets,
                       const size_t b_ld, const T* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
                       const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice) {
  try {
    ContextGuard guard(context);
    return static_cast<StatusCode>(b200blas_gemm_batched(
        DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose), static_cast<int>(b_transpose), m,
        n, k, alphas, dptr(a_buffer), a_offsets, a_ld, dptr(b_buffer), b_offsets, b_ld, betas, dptr_mut(c_buffer),
        c_offsets, c_ld, batch_count, nullptr, 0));
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

template <typename T>
StatusCode GemmStridedBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                              const size_t m, const size_t n, const size_t k, const T alpha, const CUdeviceptr a_buffer,
                              const size_t a_offset, const size_t a_ld, const size_t a_stride,
                              const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld,
                              const size_t b_stride, const T beta, CUdeviceptr c_buffer, const size_t c_offset,
                              const size_t c_ld, const size_t c_stride, const size_t batch_count,
                              const CUcontext context, const CUdevice) {
  try {
    ContextGuard guard(context);
    return static_cast<StatusCode>(b200blas_gemm_strided_batched(
        DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose), static_cast<int>(b_transpose), m,
        n, k, &alpha, dptr(a_buffer), a_offset, a_ld, a_stride, dptr(b_buffer), b_offset, b_ld, b_stride, &beta,
        dptr_mut(c_buffer), c_offset, c_ld, c_stride, batch_count, nullptr, 0));
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

template <typename T>
StatusCode GemmTempBufferSize(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                              const size_t m, const size_t n, const size_t k, const size_t a_offset, const size_t a_ld,
                              const size_t b_offset, const size_t b_ld, const size_t c_offset, const size_t c_ld,
                              const CUdevice, size_t& temp_buffer_size) {
  return static_cast<StatusCode>(b200blas_gemm_temp_buffer_size(
      DtypeOf<T>::value, static_cast<int>(layout), static_cast<int>(a_transpose), static_cast<int>(b_transpose), m, n,
      k, a_offset, a_ld, b_offset, b_ld, c_offset, c_ld, &temp_buffer_size));
}

StatusCode ClearCache() { return static_cast<StatusCode>(b200blas_clear_cache()); }
StatusCode FillCache(const CUdevice device) { return static_cast<StatusCode>(b200blas_fill_cache(device)); }

StatusCode RetrieveParameters(const CUdevice device, const std::string& kernel_name, const Precision precision,
                              std::unordered_map<std::string, size_t>& parameters) {
  try {
    size_t count = 0;
    int st = b200blas_retrieve_parameters(device, kernel_name.c_str(), static_cast<int>(precision), nullptr, nullptr,
                                          0, &count);
    if (st != 0) return static_cast<StatusCode>(st);
    std::vector<const char*> names(count);
    std::vector<size_t> values(count);
    st = b200blas_retrieve_parameters(device, kernel_name.c_str(), static_cast<int>(precision), names.data(),
                                      values.data(), count, &count);
    if (st != 0) return static_cast<StatusCode>(st);
    for (size_t i = 0; i < names.size() && i < count; ++i) parameters[names[i]] = values[i];
    return StatusCode::kSuccess;
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

StatusCode OverrideParameters(const CUdevice device, const std::string& kernel_name, const Precision precision,
                              const std::unordered_map<std::string, size_t>& parameters) {
  try {
    std::vector<const char*> names;
    std::vector<size_t> values;
    for (const auto& kv : parameters) {
      names.push_back(kv.first.c_str());
      values.push_back(kv.second);
    }
    return static_cast<StatusCode>(b200blas_override_parameters(device, kernel_name.c_str(),
                                                                static_cast<int>(precision), names.data(),
                                                                values.data(), names.size()));
  } catch (...) {
    return StatusCode::kUnexpectedError;
  }
}

// ---- exported instantiations ------------------------------------------------------------------------------

#define B200_INSTANTIATE_GEMM_FAMILY(T)                                                                               \
  template StatusCode PUBLIC_API Gemm<T>(const Layout, const Transpose, const Transpose, const size_t, const size_t,  \
                                         const size_t, const T, const CUdeviceptr, const size_t, const size_t,        \
                                         const CUdeviceptr, const size_t, const size_t, const T, CUdeviceptr,         \
                                         const size_t, const size_t, const CUcontext, const CUdevice, CUdeviceptr);   \
  template StatusCode PUBLIC_API GemmBatched<T>(const Layout, const Transpose, const Transpose, const size_t,         \
                                                const size_t, const size_t, const T*, const CUdeviceptr,              \
                                                const size_t*, const size_t, const CUdeviceptr, const size_t*,        \
                                                const size_t, const T*, CUdeviceptr, const size_t*, const size_t,     \
                                                const size_t, const CUcontext, const CUdevice);                       \
  template StatusCode PUBLIC_API GemmStridedBatched<T>(                                                               \
      const Layout, const Transpose, const Transpose, const size_t, const size_t, const size_t, const T,              \
      const CUdeviceptr, const size_t, const size_t, const size_t, const CUdeviceptr, const size_t, const size_t,     \
      const size_t, const T, CUdeviceptr, const size_t, const size_t, const size_t, const size_t, const CUcontext,    \
      const CUdevice);                                                                                                \
  template StatusCode PUBLIC_API GemmTempBufferSize<T>(const Layout, const Transpose, const Transpose, const size_t,  \
                                                       const size_t, const size_t, const size_t, const size_t,        \
                                                       const size_t, const size_t, const size_t, const size_t,        \
                                                       const CUdevice, size_t&);

#define B200_INSTANTIATE_CONV(T)                                                                                      \
  template StatusCode PUBLIC_API Convgemm<T>(const KernelMode, const size_t, const size_t, const size_t,              \
                                             const size_t, const size_t, const size_t, const size_t, const size_t,    \
                                             const size_t, const size_t, const size_t, const size_t, const size_t,    \
                                             const CUdeviceptr, const size_t, const CUdeviceptr, const size_t,        \
                                             CUdeviceptr, const size_t, const CUcontext, const CUdevice);

B200_INSTANTIATE_GEMM_FAMILY(float)
B200_INSTANTIATE_GEMM_FAMILY(double)
B200_INSTANTIATE_GEMM_FAMILY(unsigned short)
B200_INSTANTIATE_GEMM_FAMILY(std::complex<float>)
B200_INSTANTIATE_GEMM_FAMILY(std::complex<double>)
B200_INSTANTIATE_CONV(float)
B200_INSTANTIATE_CONV(double)
B200_INSTANTIATE_CONV(unsigned short)

}  // namespace clblast
