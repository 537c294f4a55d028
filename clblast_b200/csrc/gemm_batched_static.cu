// GemmBatched for callers that must not allocate device memory.
//
// clblast::GemmBatched takes its per-batch scalars and offsets as host arrays, so every call needs a small
// device table (three offsets and two scalars per batch). The regular entry point obtains that table from the
// stream-ordered allocator. Some programs cannot do that: an inference server or solver that has handed the
// whole device memory to its own arena (any further allocation fails or fragments it), or a latency-critical
// loop that must not touch the allocator's locks and implicit synchronisation. For those, this file provides
// one more entry point whose table lives in a fixed array inside the library image.
//
// Consequences of the fixed array, all part of the contract:
//   - at most kMaxBatches batches per call; larger counts are rejected with kInvalidBatchCount;
//   - every GPU that loads the library holds the array (kTableBytes, about 224 KB) until the process exits;
//   - all calls on a device share the array, and it keeps the previous call's tables: a call overwrites the part
//     it uses before its kernel starts, in stream order. Two calls whose work overlaps on the GPU (different
//     streams, or two host threads) race on it; callers must order them themselves;
//   - the first call on each device resolves the array's device address; make that call before starting any
//     stream capture.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "b200blas.h"
#include "noalloc_bridge.h"

namespace b200 {

namespace {

constexpr size_t kMaxBatches = B200BLAS_STATIC_MAX_BATCHES;
// Per batch: 3 offsets of 8 bytes + 2 scalars of up to 16 bytes (complex double), plus alignment slack.
constexpr size_t kTableBytes = kMaxBatches * (3 * 8 + 2 * 16) + 64;

// In host code this name is only a handle for the symbol, never a device address; the address is resolved once
// per device with cudaGetSymbolAddress below and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_batched_tables[kTableBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_table_address[kMaxDevices] = {nullptr};

// Device address of the table on the current device, resolved on first use with that device current.
cudaError_t table_address(unsigned char** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_table_address[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_batched_tables);
    if (err != cudaSuccess) return err;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    g_table_address[dev] = ptr;
  }
  *out = g_table_address[dev];
  return cudaSuccess;
}

}  // namespace

}  // namespace b200

extern "C" int b200blas_gemm_batched_static(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n,
                                            size_t k, const void* alphas, const void* a, const size_t* a_offsets,
                                            size_t a_ld, const void* b, const size_t* b_offsets, size_t b_ld,
                                            const void* betas, void* c, const size_t* c_offsets, size_t c_ld,
                                            size_t batch_count, void* stream, int wait) {
  using namespace b200;
  if (batch_count > kMaxBatches) {
    std::fprintf(stderr, "b200blas_gemm_batched_static: batch_count %zu exceeds the fixed table's %zu batches\n",
                 batch_count, kMaxBatches);
    return -2049;  // kInvalidBatchCount
  }
  // Host staging lives on this thread's stack; the copy below is from pageable memory, so it has been consumed
  // by the time cudaMemcpyAsync returns.
  alignas(16) unsigned char host_block[kTableBytes];
  GemmDesc desc;
  BatchedTables tables;
  const int status = prepare_batched(dtype, layout, a_transpose, b_transpose, m, n, k, alphas, a, a_offsets, a_ld, b,
                                     b_offsets, b_ld, betas, c, c_offsets, c_ld, batch_count, host_block,
                                     sizeof(host_block), &desc, &tables);
  if (status != 0) return status;

  unsigned char* device_block = nullptr;
  cudaError_t err = table_address(&device_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (err == cudaSuccess) err = cudaMemcpyAsync(device_block, host_block, tables.total, cudaMemcpyHostToDevice, s);
  if (err == cudaSuccess) {
    patch_batched_tables(&desc, tables, device_block);
    err = dispatch_desc(desc, s);
  }
  if (err == cudaSuccess && wait) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    std::fprintf(stderr, "b200blas_gemm_batched_static: CUDA error %d (%s)\n", static_cast<int>(err),
                 cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return 0;
}
