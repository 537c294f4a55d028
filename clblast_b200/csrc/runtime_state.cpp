#include "runtime_state.h"

#include <map>
#include <mutex>
#include <utility>

#include <cstring>
#include <mutex>

#include "driver_api.h"

namespace b200 {

int per_device(std::atomic<int> (&table)[kMaxDevices], int (*compute)()) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  int v = table[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  v = compute();
  if (v > 0) table[dev].store(v, std::memory_order_relaxed);  // racing threads compute the same value
  return v;
}

int sm_count() {
  static std::atomic<int> counts[kMaxDevices];
  return per_device(counts, [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return n;
  });
}

int context_key(unsigned long long* key) {
  const DriverApi& drv = driver_api();
  if (!drv.ok) return CUDA_ERROR_NOT_INITIALIZED;
  CUcontext ctx = nullptr;
  CUresult r = drv.CtxGetCurrent(&ctx);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  if (!ctx) {
    // No context is current: let the runtime bind the primary context of the current device (cudaSetDevice
    // initialises it since CUDA 12; no allocator call is involved).
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess)
      return static_cast<int>(cudaGetLastError());
    r = drv.CtxGetCurrent(&ctx);
    if (r != CUDA_SUCCESS || !ctx) return CUDA_ERROR_INVALID_CONTEXT;
  }
  unsigned long long k = reinterpret_cast<unsigned long long>(ctx);
  if (drv.CtxGetId) {
    unsigned long long id = 0;
    if (drv.CtxGetId(ctx, &id) == CUDA_SUCCESS) k = (id << 1) | 1ull;  // odd keys: ids; even keys: handle values
  }
  *key = k;
  return 0;
}

cudaError_t kernel_ready(const void* func, int smem_bytes, int* regs) {
  struct Entry { int smem; int regs; };
  static std::mutex guard;
  static std::map<std::pair<unsigned long long, const void*>, Entry> table;  // (context, kernel)
  unsigned long long ctx = 0;
  if (context_key(&ctx) != 0) ctx = 0;  // no key: fall through to the runtime calls every time
  {
    std::lock_guard<std::mutex> lock(guard);
    const auto it = table.find({ctx, func});
    if (ctx != 0 && it != table.end() && it->second.smem >= smem_bytes && (regs == nullptr || it->second.regs > 0)) {
      if (regs) *regs = it->second.regs;
      return cudaSuccess;
    }
  }
  Entry e = {smem_bytes, 0};
  if (regs) {
    cudaFuncAttributes attr;
    const cudaError_t ga = cudaFuncGetAttributes(&attr, func);
    if (ga != cudaSuccess) return ga;
    e.regs = attr.numRegs;
    *regs = attr.numRegs;
  }
  if (smem_bytes > 48 * 1024) {
    const cudaError_t sa = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (sa != cudaSuccess) return sa;
  }
  if (ctx != 0) {
    std::lock_guard<std::mutex> lock(guard);
    Entry& slot = table[{ctx, func}];
    if (slot.smem < e.smem) slot.smem = e.smem;
    if (e.regs > 0) slot.regs = e.regs;
  }
  return cudaSuccess;
}

namespace {

// One page of the library image; only the first 16 bytes are used.
alignas(4096) unsigned int g_status_page[1024];
std::once_flag g_status_once;
unsigned int* g_status_device = nullptr;

void register_status_page() {
  if (cudaHostRegister(g_status_page, sizeof(g_status_page), cudaHostRegisterPortable | cudaHostRegisterMapped) !=
      cudaSuccess) {
    cudaGetLastError();
    return;
  }
  void* dev = nullptr;
  if (cudaHostGetDevicePointer(&dev, g_status_page, 0) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  g_status_device = static_cast<unsigned int*>(dev);
}

}  // namespace

unsigned int* tc_status_device() {
  std::call_once(g_status_once, register_status_page);
  return g_status_device;
}

bool tc_status_read(unsigned int out[4], bool clear) {
  if (tc_status_device() == nullptr) return false;
  volatile unsigned int* page = g_status_page;
  for (int i = 0; i < 4; ++i) out[i] = page[i];
  if (clear && out[0] != 0) {
    for (int i = 0; i < 4; ++i) page[i] = 0;
  }
  return true;
}

}  // namespace b200
