// Internal launch interface between the C-ABI layer and the kernel translation units.
#pragma once

#include <cuda_runtime_api.h>

#include "gemm_desc.h"

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

// Reads (and optionally clears) the tensor-core kernel's device status words: out[0] != 0 means a bounded wait
// expired in some CTA (1 producer, 2 accumulator-free, 3 operands-ready, 4 accumulator-ready), out[1] is the block.
cudaError_t tc_f16_status(unsigned int out[4], bool clear);

// Shape classes of the CUDA-core family. kLarge needs enough 128x128 tiles to fill the 148 SMs.
enum class SimtClass { kSmall, kMedium, kLarge };

inline SimtClass classify_simt(const GemmDesc& d) {
  const long long mn_min = d.m < d.n ? d.m : d.n;
  if (d.force_small || mn_min <= 32) return SimtClass::kSmall;
  const long long tiles_l = ((d.m + 127) / 128) * ((d.n + 127) / 128) * d.batch;
  if (mn_min >= 96 && tiles_l >= 120) return SimtClass::kLarge;
  return SimtClass::kMedium;
}

}  // namespace b200
