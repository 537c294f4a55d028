// Large half / single GEMMs whose operands break TMA's alignment rules (a base that is not 16-byte aligned, or a
// leading dimension that is not a multiple of 16 bytes, e.g. BLAS callers that pad ld by an odd amount).
//
// The TMA-fed tensor-core kernels cannot address such an operand, and gathering it element by element inside the
// kernel runs at less than half their speed. When the product is large, each offending operand is instead copied once
// into stream-ordered scratch with an aligned pitch (one read and one write of O(n^2) data, a few per cent of the
// O(n^3) product's time) and the TMA kernels run on the copy. C is never copied: the kernels write it with plain
// stores wherever it lies. Smaller problems, batches and problems whose copy would not pay keep the in-kernel gather
// (fp32) or the CUDA-core kernel (fp16).
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "kernels/launchers.h"
#include "kernels/level3_aux.h"

namespace b200 {

cudaError_t launch_repitched(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if ((d.dtype != 16 && d.dtype != 32) || d.is_conv || d.force_small || d.batch != 1 || d.a_offs || d.conj_a || d.conj_b)
    return cudaErrorNotSupported;
  static const bool disabled = [] {  // B200BLAS_REPITCH=0: keep the in-kernel gather / the CUDA-core kernel
    const char* v = std::getenv("B200BLAS_REPITCH");
    return v != nullptr && std::strcmp(v, "0") == 0;
  }();
  if (disabled) return cudaErrorNotSupported;
  const long long elem = d.dtype == 16 ? 2 : 4, gran = 16 / elem;
  const auto misaligned = [&](const void* base, long long off, long long ld) {
    return ((reinterpret_cast<uintptr_t>(base) + static_cast<uintptr_t>(off * elem)) & 15) != 0 || (ld % gran) != 0;
  };
  const bool a_bad = misaligned(d.a, d.a_off, d.lda), b_bad = misaligned(d.b, d.b_off, d.ldb);
  if (!a_bad && !b_bad) return cudaErrorNotSupported;   // nothing to do: the regular selection serves the call
  // The copies move (m + n) k elements twice, the product does m n k multiply-adds: at m n / (m + n) = 512 the copies
  // take about half the product's time on the TMA kernels, which still beats the in-kernel gather (2.2x the product's
  // time); below that the gather is kept. Only where the tensor-core kernels would accept the problem.
  if (d.m < 512 || d.n < 256 || d.k < 128) return cudaErrorNotSupported;
  if (static_cast<double>(d.m) * d.n / static_cast<double>(d.m + d.n) < 512.0) return cudaErrorNotSupported;

  // memory-order extents of the two operands: `one` contiguous elements per line, `two` lines
  const long long a_one = d.a_kcontig ? d.k : d.m, a_two = d.a_kcontig ? d.m : d.k;
  const long long b_one = d.b_kcontig ? d.k : d.n, b_two = d.b_kcontig ? d.n : d.k;
  const long long a_pitch = (a_one + gran - 1) / gran * gran, b_pitch = (b_one + gran - 1) / gran * gran;
  const size_t a_bytes = a_bad ? static_cast<size_t>(a_pitch) * a_two * elem : 0;
  const size_t a_slot = (a_bytes + 255) / 256 * 256;
  const size_t b_bytes = b_bad ? static_cast<size_t>(b_pitch) * b_two * elem : 0;
  unsigned char* scratch = nullptr;
  cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&scratch), a_slot + b_bytes + 256, stream);
  if (err != cudaSuccess) return err;
  GemmDesc r = d;
  RepitchJob jobs[2] = {};
  if (a_bad) {
    jobs[0] = {static_cast<const unsigned char*>(d.a) + d.a_off * elem, scratch, a_one, a_two, d.lda, a_pitch};
    r.a = scratch; r.a_off = 0; r.lda = a_pitch;
  }
  if (b_bad) {
    jobs[1] = {static_cast<const unsigned char*>(d.b) + d.b_off * elem, scratch + a_slot, b_one, b_two, d.ldb, b_pitch};
    r.b = scratch + a_slot; r.b_off = 0; r.ldb = b_pitch;
  }
  err = launch_repitch(static_cast<int>(elem), jobs, stream);
  if (err == cudaSuccess) {
    const char* inner = "none";
    if (d.dtype == 16) {
      err = launch_tc_f16_pair(r, stream, &inner);
      if (err == cudaErrorNotSupported) err = launch_tc_f16(r, stream, &inner);
    } else {
      err = launch_tc_f32_pair(r, stream, &inner);
      if (err == cudaErrorNotSupported) err = launch_tc_f32(r, stream, &inner);
    }
    static thread_local char label[96];
    std::snprintf(label, sizeof(label), "repitched_%s", inner);
    *name = label;
  }
  const cudaError_t ferr = cudaFreeAsync(scratch, stream);
  return err != cudaSuccess ? err : ferr;
}

}  // namespace b200
