// CUDA-core GEMM instantiations and the static tile-selection table for dtype c64.
#include "gemm_simt.cuh"
#include "launchers.h"

namespace b200 {

cudaError_t launch_simt_c64(const GemmDesc& d, cudaStream_t stream, const char** name) {
  using Large = SimtLauncher<TraitsC64, 64, 64, 8, 4, 4, 1>;
  using Medium = SimtLauncher<TraitsC64, 64, 64, 8, 4, 4, 1>;
  using Small = SimtLauncher<TraitsC64, 32, 32, 8, 4, 4, 2>;
  const SimtClass cls = classify_simt(d);

  switch (cls) {
    case SimtClass::kLarge: *name = "simt_c64_large"; return Large::launch(d, stream);
    case SimtClass::kMedium: *name = "simt_c64_medium"; return Medium::launch(d, stream);
    default: *name = "simt_c64_small"; return Small::launch(d, stream);
  }
}

}  // namespace b200
