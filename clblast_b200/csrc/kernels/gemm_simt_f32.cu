// CUDA-core GEMM instantiations and the static tile-selection table for dtype f32.
#include "gemm_simt.cuh"
#include "launchers.h"

namespace b200 {

cudaError_t launch_simt_f32(const GemmDesc& d, cudaStream_t stream, const char** name) {
  static const SimtConfig table[] = {
      {128, 128, 1.0, 1, false},
      {64, 128, 0.85, 1, false},
      {64, 64, 0.7, 2, false},
      {32, 32, 0.5, 8, true},
  };
  switch (pick_simt(d, table, 4)) {
    case 0:
      if (d.is_conv) { *name = "conv_simt_f32_128x128"; return SimtLauncher<TraitsF32, 128, 128, 16, 8, 8, 2, 1>::launch_conv(d, stream); }
      *name = "simt_f32_128x128"; return SimtLauncher<TraitsF32, 128, 128, 16, 8, 8, 2, 1>::launch(d, stream);
    case 1:
      if (d.is_conv) { *name = "conv_simt_f32_64x128"; return SimtLauncher<TraitsF32, 64, 128, 16, 8, 8, 3, 1>::launch_conv(d, stream); }
      *name = "simt_f32_64x128"; return SimtLauncher<TraitsF32, 64, 128, 16, 8, 8, 3, 1>::launch(d, stream);
    case 2:
      if (d.is_conv) { *name = "conv_simt_f32_64x64"; return SimtLauncher<TraitsF32, 64, 64, 16, 8, 8, 3, 2>::launch_conv(d, stream); }
      *name = "simt_f32_64x64"; return SimtLauncher<TraitsF32, 64, 64, 16, 8, 8, 3, 2>::launch(d, stream);
    default:
      if (d.is_conv) { *name = "conv_simt_f32_32x32"; return SimtLauncher<TraitsF32, 32, 32, 8, 8, 8, 3, 8>::launch_conv(d, stream); }
      *name = "simt_f32_32x32"; return SimtLauncher<TraitsF32, 32, 32, 8, 8, 8, 3, 8>::launch(d, stream);
  }
}

}  // namespace b200
