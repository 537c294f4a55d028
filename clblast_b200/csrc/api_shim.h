// Shared by the translation units that export the reference's C++ API: element-type codes, the context guard and
// pointer casts.
#pragma once

#include <complex>

#include "clblast_cuda.h"
#include "driver_api.h"

namespace clblast {
namespace shim {

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = 32; };
template <> struct DtypeOf<double> { static constexpr int value = 64; };
template <> struct DtypeOf<unsigned short> { static constexpr int value = 16; };
template <> struct DtypeOf<std::complex<float>> { static constexpr int value = 3232; };
template <> struct DtypeOf<std::complex<double>> { static constexpr int value = 6464; };

// The reference requires `context` to be current on the calling thread and never switches contexts itself
// (src/cupp11.hpp:374). This guard keeps that working and additionally tolerates a caller whose thread has a
// different context current, by pushing the given one for the duration of the call.
class ContextGuard {
 public:
  explicit ContextGuard(CUcontext wanted) : pushed_(false) {
    const b200::DriverApi& drv = b200::driver_api();
    if (!drv.ok || !wanted) return;
    CUcontext current = nullptr;
    if (drv.CtxGetCurrent(&current) == CUDA_SUCCESS && current != wanted) {
      pushed_ = (drv.CtxPushCurrent(wanted) == CUDA_SUCCESS);
    }
  }
  ~ContextGuard() {
    if (pushed_) {
      CUcontext dummy = nullptr;
      b200::driver_api().CtxPopCurrent(&dummy);
    }
  }

 private:
  bool pushed_;
};

inline const void* dptr(CUdeviceptr p) { return reinterpret_cast<const void*>(p); }
inline void* dptr_mut(CUdeviceptr p) { return reinterpret_cast<void*>(p); }


}  // namespace shim
using namespace shim;
}  // namespace clblast
