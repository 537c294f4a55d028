// Lazily bound CUDA driver entry points.
//
// The library links the CUDA runtime statically and binds the handful of driver calls it needs from
// libcuda.so.1 at first use, so the shared object can be loaded (and its symbol table inspected) on a machine
// without a driver; any compute call there fails with CUDA_ERROR_NOT_INITIALIZED instead of computing on the host.
#pragma once

#include <cuda.h>

namespace b200 {

struct DriverApi {
  CUresult (*CtxGetCurrent)(CUcontext*);
  CUresult (*CtxPushCurrent)(CUcontext);
  CUresult (*CtxPopCurrent)(CUcontext*);
  CUresult (*CtxGetId)(CUcontext, unsigned long long*);  // may be null on old drivers
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
  CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  // Stream memory operations (used by the multi-GPU helpers only; may be null on old drivers).
  CUresult (*StreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  CUresult (*StreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
  bool ok;
};

// Returns the bound table; `ok` is false when libcuda.so.1 or one of the symbols is missing.
const DriverApi& driver_api();

}  // namespace b200
