// Large complex GEMMs on the real-valued tensor-core kernels.
//
// C = alpha * op(A) * op(B) + beta * C with complex m x k, k x n and m x n matrices is the real product
//   C^ (2m x n) = A^ (2m x 2k) * B^ (2k x n)
// where C^ and B^ are the interleaved (re, im) memory of C and op(B) read as real matrices with doubled leading
// dimension, and A^ holds, for every element z = alpha * op(A)(i, l), the 2 x 2 block [[Re z, -Im z], [Im z, Re z]]:
// column 2l of A^ is column l of alpha * op(A) in interleaved form, column 2l + 1 is the same column times i.
// The real product has the flop count of the complex one (8 m n k) and runs on the error-compensated 3xTF32 kernels
// (complex single) or the FP64 tensor-core kernel (complex double) instead of the 64 x 64 CUDA-core kernel.
//
// A^ is written by two scaled copies (alpha and i * alpha) into stream-ordered scratch; op(B) is used where it lies
// when it is K-contiguous and not conjugated, else packed by one more copy; a complex beta scales C in place first
// (a real beta goes straight into the product). Replaces, for large problems, the reference's complex instantiations of
// the Xgemm kernel (src/kernels/level3/xgemm_part3.opencl:53-305 with PRECISION 3232 / 6464).
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "host_common.h"
#include "kernels/launchers.h"
#include "kernels/level3_aux.h"

namespace b200 {

cudaError_t launch_complex_on_real(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if ((d.dtype != 3232 && d.dtype != 6464) || d.is_conv || d.force_small || d.tri || d.batch != 1 || d.a_offs)
    return cudaErrorNotSupported;
  static const bool forced_simt = [] {
    const char* v = std::getenv("B200BLAS_CGEMM");
    return v != nullptr && std::strcmp(v, "simt") == 0;
  }();
  if (forced_simt) return cudaErrorNotSupported;
  const bool single = d.dtype == 3232;
  const long long m2 = 2 * d.m, k2 = 2 * d.k;
  if (m2 > 0x7FFFFFFF || d.n > 0x7FFFFFFF || k2 > 0x7FFFFFFF) return cudaErrorNotSupported;
  // Sizes at which the real problem is certain to be accepted by the tensor-core launchers below.
  if (single) {
    if (m2 < 512 || d.n < 256 || k2 < 256 || static_cast<double>(m2) * d.n * k2 < 4.0 * 134217728.0)
      return cudaErrorNotSupported;
  } else {
    const long long tiles = ((m2 + 127) / 128) * ((d.n + 127) / 128);
    if (m2 < 256 || d.n < 128 || k2 < 64 || tiles < 148) return cudaErrorNotSupported;
  }
  const size_t real_bytes = single ? 4 : 8;
  const bool pack_b = !d.b_kcontig || d.conj_b;
  const size_t a_hat_bytes = static_cast<size_t>(m2) * k2 * real_bytes;
  const size_t b_hat_bytes = pack_b ? static_cast<size_t>(k2) * d.n * real_bytes : 0;
  unsigned char* scratch = nullptr;
  cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&scratch), a_hat_bytes + b_hat_bytes + 256, stream);
  if (err != cudaSuccess) return err;
  unsigned char* a_hat = scratch;
  unsigned char* b_hat = scratch + ((a_hat_bytes + 255) / 256) * 256;

  // A^: even columns alpha * op(A), odd columns i * alpha * op(A); as a complex matrix its leading dimension is 2m and
  // the odd columns start m elements in. The source is read in memory order: `one` is its contiguous extent.
  const double i_alpha[2] = {-d.alpha[1], d.alpha[0]};
  const long long a_one = d.a_kcontig ? d.k : d.m, a_two = d.a_kcontig ? d.m : d.k;
  err = launch_omatcopy(d.dtype, d.a_kcontig != 0, d.conj_a != 0, a_one, a_two, d.alpha, d.a, d.a_off, d.lda, a_hat, 0, m2,
                        stream);
  if (err == cudaSuccess)
    err = launch_omatcopy(d.dtype, d.a_kcontig != 0, d.conj_a != 0, a_one, a_two, i_alpha, d.a, d.a_off, d.lda, a_hat,
                          d.m, m2, stream);
  const double one[2] = {1.0, 0.0};
  if (err == cudaSuccess && pack_b) {
    const long long b_one = d.b_kcontig ? d.k : d.n, b_two = d.b_kcontig ? d.n : d.k;
    err = launch_omatcopy(d.dtype, !d.b_kcontig, d.conj_b != 0, b_one, b_two, one, d.b, d.b_off, d.ldb, b_hat, 0, d.k,
                          stream);
  }
  double beta_real = d.beta[0];
  if (err == cudaSuccess && d.beta[1] != 0.0) {   // complex beta: C = beta * C in place, then the product adds to it
    err = launch_omatcopy(d.dtype, false, false, d.m, d.n, d.beta, d.c, d.c_off, d.ldc, d.c, d.c_off, d.ldc, stream);
    beta_real = 1.0;
  }
  if (err == cudaSuccess) {
    GemmDesc r = {};
    r.dtype = single ? 32 : 64;
    r.m = m2; r.n = d.n; r.k = k2;
    r.a = a_hat; r.a_off = 0; r.lda = m2; r.a_kcontig = 0;
    if (pack_b) {
      r.b = b_hat; r.b_off = 0; r.ldb = k2;
    } else {
      r.b = d.b; r.b_off = 2 * d.b_off; r.ldb = 2 * d.ldb;
    }
    r.b_kcontig = 1;
    r.c = d.c; r.c_off = 2 * d.c_off; r.ldc = 2 * d.ldc;
    r.batch = 1;
    r.alpha[0] = 1.0;
    r.beta[0] = beta_real;
    const char* real_name = "none";
    if (single) {
      err = launch_tc_f32_pair(r, stream, &real_name);
      if (err == cudaErrorNotSupported) err = launch_tc_f32(r, stream, &real_name);
      if (err == cudaErrorNotSupported) err = launch_simt_f32(r, stream, &real_name);
    } else {
      err = launch_dmma_f64(r, stream, &real_name);
      if (err == cudaErrorNotSupported) err = launch_simt_f64(r, stream, &real_name);
    }
    static thread_local char label[96];
    std::snprintf(label, sizeof(label), "complex_on_%s", real_name);
    *name = label;
  }
  const cudaError_t ferr = cudaFreeAsync(scratch, stream);
  return err != cudaSuccess ? err : ferr;
}

}  // namespace b200
