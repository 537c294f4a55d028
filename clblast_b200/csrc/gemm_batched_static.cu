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
//   - the first call under each context resolves the array's device address in that context;
//   - the call is refused (kUnexpectedError, nothing enqueued) on a stream that is being captured: the host block
//     its table copy reads is reused by the next call.
#include <cuda_runtime.h>

#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <new>

#include "b200blas.h"
#include "noalloc_bridge.h"
#include "runtime_state.h"

namespace b200 {

namespace {

constexpr size_t kMaxBatches = B200BLAS_STATIC_MAX_BATCHES;
// Per batch: 3 offsets of 8 bytes + 2 scalars of up to 16 bytes (complex double), plus alignment slack.
constexpr size_t kTableBytes = kMaxBatches * (3 * 8 + 2 * 16) + 64;

// In host code this name is only a handle for the symbol, never a device address; the address is resolved once
// per context with cudaGetSymbolAddress below and that pointer is what kernels receive.
static __device__ __align__(256) unsigned char g_batched_tables[kTableBytes];

// The symbol's address belongs to a context, not to a device ordinal: a process that drives one GPU through several
// contexts (CLBlast callers pass contexts made with cuCtxCreate) gets one copy of the array per context. Addresses
// are therefore cached under the same context key the library's private streams use.
std::mutex g_setup_mutex;
std::map<unsigned long long, unsigned char*> g_table_address;

// Device address of the table in the current context, resolved on the first call made under that context.
cudaError_t table_address(unsigned char** out) {
  unsigned long long key = 0;
  if (context_key(&key) != 0) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  auto it = g_table_address.find(key);
  if (it == g_table_address.end()) {
    unsigned char* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_batched_tables);
    if (err != cudaSuccess) return err;
    if (ptr == nullptr) return cudaErrorInvalidSymbol;
    it = g_table_address.emplace(key, ptr).first;
  }
  *out = it->second;
  return cudaSuccess;
}

// Host staging block of the calling thread (host memory, kept for the thread's lifetime): the tables are far too
// large for the small stacks of worker threads that language runtimes create.
unsigned char* host_staging() {
  thread_local std::unique_ptr<unsigned char[]> block;
  if (!block) block.reset(new (std::nothrow) unsigned char[kTableBytes]);
  return block.get();
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
  // A capturing stream is refused before anything is enqueued: the table copy below reads a host block that is
  // rewritten by the next call, so a graph holding that copy would replay stale tables.
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    std::fprintf(stderr, "b200blas_gemm_batched_static: the stream is being captured; the call is refused\n");
    return -2039;  // kUnexpectedError
  }
  // The copy below is from pageable memory, so the block has been consumed by the time cudaMemcpyAsync returns
  // and the thread's next call may overwrite it.
  unsigned char* const host_block = host_staging();
  if (host_block == nullptr) return -2039;
  GemmDesc desc;
  BatchedTables tables;
  const int status = prepare_batched(dtype, layout, a_transpose, b_transpose, m, n, k, alphas, a, a_offsets, a_ld, b,
                                     b_offsets, b_ld, betas, c, c_offsets, c_ld, batch_count, host_block, kTableBytes,
                                     &desc, &tables);
  if (status != 0) return status;

  unsigned char* device_block = nullptr;
  cudaError_t err = table_address(&device_block);
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
  // With `wait` the stream has finished: report a tensor-core kernel whose bounded wait expired.
  return wait ? status_after_sync() : 0;
}
