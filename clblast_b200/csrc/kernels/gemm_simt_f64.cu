// CUDA-core GEMM instantiations and the static tile-selection table for dtype f64.
#include "gemm_simt.cuh"
#include "launchers.h"

namespace b200 {

cudaError_t launch_simt_f64(const GemmDesc& d, cudaStream_t stream, const char** name) {
  static const SimtConfig table[] = {
      {128, 128, 1.0, 1, false},
      {64, 128, 0.85, 1, false},
      {64, 64, 0.7, 2, false},
      {32, 32, 0.5, 4, true},
  };
  switch (pick_simt(d, table, 4)) {
    case 0:
      if (d.is_conv) { *name = "conv_simt_f64_128x128"; return SimtLauncher<TraitsF64, 128, 128, 8, 8, 8, 1, 1>::launch_conv(d, stream); }
      *name = "simt_f64_128x128"; return SimtLauncher<TraitsF64, 128, 128, 8, 8, 8, 1, 1>::launch(d, stream);
    case 1:
      if (d.is_conv) { *name = "conv_simt_f64_64x128"; return SimtLauncher<TraitsF64, 64, 128, 8, 8, 8, 2, 1>::launch_conv(d, stream); }
      *name = "simt_f64_64x128"; return SimtLauncher<TraitsF64, 64, 128, 8, 8, 8, 2, 1>::launch(d, stream);
    case 2:
      if (d.is_conv) { *name = "conv_simt_f64_64x64"; return SimtLauncher<TraitsF64, 64, 64, 8, 8, 8, 2, 2>::launch_conv(d, stream); }
      *name = "simt_f64_64x64"; return SimtLauncher<TraitsF64, 64, 64, 8, 8, 8, 2, 2>::launch(d, stream);
    default:
      if (d.is_conv) { *name = "conv_simt_f64_32x32"; return SimtLauncher<TraitsF64, 32, 32, 8, 8, 8, 4, 4>::launch_conv(d, stream); }
      *name = "simt_f64_32x32"; return SimtLauncher<TraitsF64, 32, 32, 8, 8, 8, 4, 4>::launch(d, stream);
  }
}

}  // namespace b200
