// CUDA-core GEMM instantiations and the static tile-selection table for dtype c32.
#include "gemm_simt.cuh"
#include "launchers.h"

namespace b200 {

cudaError_t launch_simt_c32(const GemmDesc& d, cudaStream_t stream, const char** name) {
  static const SimtConfig table[] = {
      {64, 64, 1.0, 1, false},
      {32, 32, 0.6, 1, true},
  };
  switch (pick_simt(d, table, 2)) {
    case 0: *name = "simt_c32_64x64"; return SimtLauncher<TraitsC32, 64, 64, 8, 4, 4, 2, 1>::launch(d, stream);
    default: *name = "simt_c32_32x32"; return SimtLauncher<TraitsC32, 32, 32, 8, 4, 4, 4, 1>::launch(d, stream);
  }
}

}  // namespace b200
