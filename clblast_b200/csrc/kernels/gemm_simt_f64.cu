// CUDA-core GEMM instantiations and the static tile-selection table for dtype f64.
#include "gemm_simt.cuh"
#include "launchers.h"

namespace b200 {

cudaError_t launch_simt_f64(const GemmDesc& d, cudaStream_t stream, const char** name) {
  using Large = SimtLauncher<TraitsF64, 128, 128, 8, 8, 8, 1>;
  using Medium = SimtLauncher<TraitsF64, 64, 64, 8, 4, 4, 2>;
  using Small = SimtLauncher<TraitsF64, 32, 32, 8, 4, 4, 4>;
  const SimtClass cls = classify_simt(d);
  if (d.is_conv) {
    if (cls == SimtClass::kLarge) { *name = "conv_simt_large"; return Large::launch_conv(d, stream); }
    if (cls == SimtClass::kMedium) { *name = "conv_simt_medium"; return Medium::launch_conv(d, stream); }
    *name = "conv_simt_small"; return Small::launch_conv(d, stream);
  }
  switch (cls) {
    case SimtClass::kLarge: *name = "simt_f64_large"; return Large::launch(d, stream);
    case SimtClass::kMedium: *name = "simt_f64_medium"; return Medium::launch(d, stream);
    default: *name = "simt_f64_small"; return Small::launch(d, stream);
  }
}

}  // namespace b200
