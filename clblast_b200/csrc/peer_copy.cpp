// Building blocks for moving an operand between the GPUs of one node with the copy engines instead of a collective
// kernel: export / open of device allocations across processes, stream-ordered copies into a peer's memory, and
// stream-ordered waits on a 32-bit flag in local memory.
//
// The sharded GEMM of this library needs one exchange step: every rank must hold the whole operand that is not
// split (clblast_b200/multi_gpu.py). A collective kernel would take SMs away from the persistent GEMM kernels,
// which occupy every SM for the whole launch; copies issued with cudaMemcpyAsync run on the copy engines and flags
// are waited for by the stream front-end, so the GEMM keeps all SMs. Kernels never touch a peer's memory: data
// arrives in local memory first, then the local GEMM reads it. No counterpart in the reference, which is a
// single-device library.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstdio>
#include <cstring>

#include "b200blas.h"
#include "driver_api.h"

namespace {

int fail(const char* what, cudaError_t e) {
  std::fprintf(stderr, "b200blas: %s failed: %d (%s)\n", what, static_cast<int>(e), cudaGetErrorString(e));
  return static_cast<int>(e);
}

}  // namespace

extern "C" int b200blas_ipc_export(const void* device_ptr, unsigned char handle[64], size_t* offset) {
  if (!device_ptr || !handle || !offset) return -2039;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  const b200::DriverApi& drv = b200::driver_api();
  if (!drv.ok) return CUDA_ERROR_NOT_INITIALIZED;
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = drv.MemGetAddressRange(&base, &size, reinterpret_cast<CUdeviceptr>(device_ptr));
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail("cudaIpcGetMemHandle", e);
  }
  std::memcpy(handle, &h, 64);
  *offset = reinterpret_cast<CUdeviceptr>(device_ptr) - base;
  return 0;
}

extern "C" int b200blas_ipc_open(const unsigned char handle[64], size_t offset, void** device_ptr) {
  if (!handle || !device_ptr) return -2039;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void* base = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail("cudaIpcOpenMemHandle", e);
  }
  *device_ptr = static_cast<unsigned char*>(base) + offset;
  return 0;
}

extern "C" int b200blas_ipc_close(void* device_ptr, size_t offset) {
  if (!device_ptr) return 0;
  const cudaError_t e = cudaIpcCloseMemHandle(static_cast<unsigned char*>(device_ptr) - offset);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(e);
  }
  return 0;
}

extern "C" int b200blas_stream_copy(void* stream, void* dst, const void* src, size_t bytes) {
  if (bytes == 0) return 0;
  if (!dst || !src) return -2039;
  const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail("cudaMemcpyAsync", e);
  }
  return 0;
}

extern "C" int b200blas_stream_wait_flag(void* stream, const void* flag, uint32_t value) {
  const b200::DriverApi& drv = b200::driver_api();
  if (!drv.ok || !drv.StreamWaitValue32) return CUDA_ERROR_NOT_SUPPORTED;
  if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) return -2039;
  const CUresult r = drv.StreamWaitValue32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value,
                                           CU_STREAM_WAIT_VALUE_GEQ);
  return static_cast<int>(r);
}

extern "C" int b200blas_stream_write_flag(void* stream, void* flag, uint32_t value) {
  const b200::DriverApi& drv = b200::driver_api();
  if (!drv.ok || !drv.StreamWriteValue32) return CUDA_ERROR_NOT_SUPPORTED;
  if (!flag || (reinterpret_cast<uintptr_t>(flag) & 3)) return -2039;
  const CUresult r = drv.StreamWriteValue32(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(flag), value,
                                            CU_STREAM_WRITE_VALUE_DEFAULT);
  return static_cast<int>(r);
}
