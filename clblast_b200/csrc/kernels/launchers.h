// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once

#include <cuda_runtime_api.h>

#include "gemm_desc.h"
#include "../runtime_state.h"

namespace b200 {

// Each launcher picks a tile configuration from its static table, enqueues one kernel on `stream` and
// stores the name of the chosen kernel family in *name.
cudaError_t launch_simt_f32(const GemmDesc& d, cudaStream_t stream, const char** name);
cudaError_t launch_simt_f64(const GemmDesc& d, cudaStream_t stream, const char** name);
cudaError_t launch_simt_f16(const GemmDesc& d, cudaStream_t stream, const char** name);
cudaError_t launch_simt_c32(const GemmDesc& d, cudaStream_t stream, const char** name);
cudaError_t launch_simt_c64(const GemmDesc& d, cudaStream_t stream, const char** name);

// Tensor-core HGEMM (TMA + tcgen05 + TMEM). Returns cudaErrorNotSupported, without launching anything, when
// the call does not meet the kernel's layout and alignment requirements; the caller then uses the CUDA-core path.
cudaError_t launch_tc_f16(const GemmDesc& d, cudaStream_t stream, const char** name);
// The same on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles shared by two SMs), tried first.
cudaError_t launch_tc_f16_pair(const GemmDesc& d, cudaStream_t stream, const char** name);

// DGEMM on the FP64 tensor-core instructions (mma.sync m8n8k4). Same contract as launch_tc_f16.
cudaError_t launch_dmma_f64(const GemmDesc& d, cudaStream_t stream, const char** name);

// Tensor-core SGEMM (error-compensated 3xTF32). Same contract as launch_tc_f16.
cudaError_t launch_tc_f32(const GemmDesc& d, cudaStream_t stream, const char** name);

// The same on CTA pairs (256 x 256 tiles shared by two SMs), tried first for large problems.
cudaError_t launch_tc_f32_pair(const GemmDesc& d, cudaStream_t stream, const char** name);

// Batches of narrow problems (at most 64 rows) on the same kernel, computed as the transposed problem.
cudaError_t launch_tc_f32_narrow(const GemmDesc& d, cudaStream_t stream, const char** name);
// Tensor-core Convgemm (same kernel, op(A) gathered from the image by the split warps).
cudaError_t launch_tc_conv_f32(const GemmDesc& d, cudaStream_t stream, const char** name);

// Streaming kernel for large batches of small fp32 problems (cp.async double buffering across the batch). Returns
// cudaErrorNotSupported without launching when the call does not meet its shape and alignment requirements.
cudaError_t launch_small_batched_f32(const GemmDesc& d, cudaStream_t stream, const char** name);

// Large single complex GEMMs as a real product of twice the rows and twice the inner dimension on the kernels above
// (csrc/complex_on_real.cpp). Same contract as launch_tc_f16.
cudaError_t launch_complex_on_real(const GemmDesc& d, cudaStream_t stream, const char** name);

// Half / double Convgemm as im2col into scratch plus one strided-batched GEMM on the tensor-core kernels
// (csrc/conv_two_step.cpp). Same contract as launch_tc_f16.
cudaError_t launch_conv_two_step(const GemmDesc& d, cudaStream_t stream, const char** name);
// Half-precision Convgemm as an implicit GEMM with the im2col matrix in tensor memory (gemm_tc_f16_conv.cu).
cudaError_t launch_tc_conv_f16(const GemmDesc& d, cudaStream_t stream, const char** name);
// Double-precision Convgemm as an implicit GEMM on the FP64 mma.sync kernel (gemm_dmma_f64.cu).
cudaError_t launch_dmma_conv_f64(const GemmDesc& d, cudaStream_t stream, const char** name);

// Large half / single GEMMs with operands TMA cannot address: the offending operands are copied once into scratch with
// an aligned pitch and the kernels above run on the copies (csrc/repitch.cpp). Same contract as launch_tc_f16.
cudaError_t launch_repitched(const GemmDesc& d, cudaStream_t stream, const char** name);

// Number of SMs persistent kernels may occupy (0 = all); set through b200blas_set_sm_budget.
int sm_budget();

// One tile configuration of the CUDA-core family as seen by the selection table.
struct SimtConfig {
  int bm, bn;      // tile extents
  double eff;      // relative arithmetic efficiency of the configuration on full tiles (1.0 = the 128x128 tile)
  int groups;      // tiles per CTA
  bool smallest;   // the configuration forced by GemmRoutine/XGEMM_MIN_INDIRECT_SIZE
};

// Static selection: the configuration with the best (efficiency x useful fraction of the padded tiles x SM fill).
inline int pick_simt(const GemmDesc& d, const SimtConfig* cfgs, int count) {
  double ctas[8], quality[8];
  double most_ctas = 0.0;
  if (count > 8) count = 8;
  for (int i = 0; i < count; ++i) {
    if (d.force_small && cfgs[i].smallest) return i;
    const double tiles = static_cast<double>((d.m + cfgs[i].bm - 1) / cfgs[i].bm) *
                         static_cast<double>((d.n + cfgs[i].bn - 1) / cfgs[i].bn) * static_cast<double>(d.batch);
    const double useful = (static_cast<double>(d.m) * d.n * d.batch) / (tiles * cfgs[i].bm * cfgs[i].bn);
    quality[i] = cfgs[i].eff * useful;
    ctas[i] = tiles / cfgs[i].groups;
    if (ctas[i] > most_ctas) most_ctas = ctas[i];
  }
  // A problem too small to fill the SMs with any configuration is latency-bound: only padding matters then.
  const double sms = sm_count() > 0 ? sm_count() : 148.0;
  const bool tiny = most_ctas < sms;
  int best = 0;
  double best_score = -1.0;
  for (int i = 0; i < count; ++i) {
    const double fill = (tiny || ctas[i] >= sms) ? 1.0 : ctas[i] / sms;
    const double score = quality[i] * fill;
    if (score > best_score) {
      best_score = score;
      best = i;
    }
  }
  return best;
}

}  // namespace b200
