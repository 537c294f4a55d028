// Half- and double-precision Convgemm at speed: the column matrix of a group of images is written to stream-ordered
// scratch (one pass at HBM speed) and multiplied by the weights with one strided-batched GEMM on the tensor-core kernels
// (tcgen05 kind::f16 for half, the FP64 mma.sync kernel for double). The reference offers the same two-step route as
// its second convolution method (Im2col, then GEMM: src/routines/levelx/xconvgemm.cpp:24-30,96-112); single precision
// keeps the fused implicit-GEMM kernel of gemm_tc_f32.cu. Scratch is bounded: images are processed in groups whose
// column matrices take at most 256 MB.
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "kernels/launchers.h"
#include "kernels/level3_aux.h"

namespace b200 {

cudaError_t launch_conv_two_step(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (!d.is_conv || (d.dtype != 16 && d.dtype != 64) || d.force_small) return cudaErrorNotSupported;
  static const bool forced_simt = [] {
    const char* v = std::getenv("B200BLAS_CONV");
    return v != nullptr && std::strcmp(v, "simt") == 0;
  }();
  if (forced_simt) return cudaErrorNotSupported;
  const long long m = d.m, n = d.n, k = d.k, batch = d.batch;   // pixels, filters, channels * taps, images
  if (m < 128 || n < 64 || k < 32) return cudaErrorNotSupported;
  if (static_cast<double>(m) * n * k * batch < 134217728.0) return cudaErrorNotSupported;
  const size_t elem = d.dtype == 16 ? 2 : 8;
  const size_t per_image = static_cast<size_t>(k) * m * elem;
  const long long group = std::max<long long>(1, std::min<long long>(batch, (256u << 20) / per_image));
  void* col = nullptr;
  cudaError_t err = cudaMallocAsync(&col, per_image * group, stream);
  if (err != cudaSuccess) return err;
  const int out_h = static_cast<int>(m / d.conv.out_w);
  const char* gemm_name = "none";
  for (long long first = 0; first < batch && err == cudaSuccess; first += group) {
    const long long images = std::min(group, batch - first);
    err = launch_im2col(d.dtype, d.conv, out_h, d.a, d.a_off + first * d.a_stride, col, 0, stream, images, d.a_stride);
    if (err != cudaSuccess) break;
    GemmDesc g = {};
    g.dtype = d.dtype;
    g.m = m; g.n = n; g.k = k;
    g.a = col; g.a_off = 0; g.lda = m; g.a_kcontig = 0; g.a_stride = k * m;   // column matrix: pixels contiguous
    g.b = d.b; g.b_off = d.b_off; g.ldb = k; g.b_kcontig = 1; g.b_stride = 0; // weights [filter][k], shared by all images
    g.c = d.c; g.c_off = d.c_off + first * d.c_stride; g.ldc = m; g.c_stride = d.c_stride;
    g.batch = images;
    g.alpha[0] = 1.0;
    if (d.dtype == 16) {
      err = launch_tc_f16_pair(g, stream, &gemm_name);
      if (err == cudaErrorNotSupported) err = launch_tc_f16(g, stream, &gemm_name);
      if (err == cudaErrorNotSupported) err = launch_simt_f16(g, stream, &gemm_name);
    } else {
      err = launch_dmma_f64(g, stream, &gemm_name);
      if (err == cudaErrorNotSupported) err = launch_simt_f64(g, stream, &gemm_name);
    }
  }
  static thread_local char label[96];
  std::snprintf(label, sizeof(label), "conv_im2col_%s", gemm_name);
  *name = label;
  const cudaError_t ferr = cudaFreeAsync(col, stream);
  return err != cudaSuccess ? err : ferr;
}

}  // namespace b200
