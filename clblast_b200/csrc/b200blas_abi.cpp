// The C ABI of the library: argument checks, layout normalisation, kernel selection and launch.
//
// Host logic mirrored from the reference (behaviour, not code):
//   - order and meaning of the argument checks: src/routines/level3/xgemm.cpp:57-94,
//     src/routines/level3/xgemm.hpp:72-108, src/utilities/buffer_test.hpp:27-73,170-218,
//     src/routines/levelx/xgemmbatched.cpp:59-85, xgemmstridedbatched.cpp:59-90, xconvgemm.cpp:50-112;
//   - host-synchronous completion on a private non-blocking stream: src/cupp11.hpp:494-505,771-773.
// What is gone: the JIT/program cache, the tuning database lookups, the direct/indirect split with its
// padded temporaries, and the per-call stream creation and device allocations.
#include "b200blas.h"

#include <cuda_runtime_api.h>

#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "driver_api.h"
#include "kernels/launchers.h"
#include "noalloc_bridge.h"
#include "params_store.h"
#include "runtime_state.h"
#include "host_common.h"

namespace b200 {

// Upper bound on batch_count of the offset-table form: the staged tables take 56 bytes per batch, so this is 3.5 GB
// of tables; anything larger is a corrupt argument rather than a workload.
constexpr size_t kMaxBatchCount = size_t(1) << 26;

namespace {
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_sm_budget{0};
thread_local const char* t_last_kernel = "none";
}  // namespace

size_t dtype_size(int dtype) {
  switch (dtype) {
    case 16: return 2;
    case 32: return 4;
    case 64: return 8;
    case 3232: return 8;
    case 6464: return 16;
    default: return 0;
  }
}

float half_bits_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      bits = sign | ((127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// Reads one host scalar of `dtype` into (re, im) doubles.
void read_scalar(int dtype, const void* p, size_t index, double out[2]) {
  out[0] = out[1] = 0.0;
  switch (dtype) {
    case 16: out[0] = half_bits_to_float(static_cast<const uint16_t*>(p)[index]); break;
    case 32: out[0] = static_cast<const float*>(p)[index]; break;
    case 64: out[0] = static_cast<const double*>(p)[index]; break;
    case 3232:
      out[0] = static_cast<const float*>(p)[2 * index];
      out[1] = static_cast<const float*>(p)[2 * index + 1];
      break;
    case 6464:
      out[0] = static_cast<const double*>(p)[2 * index];
      out[1] = static_cast<const double*>(p)[2 * index + 1];
      break;
  }
}

// Bytes from `ptr` to the end of the device allocation that contains it. The reference compares against the
// size of the whole allocation (src/cupp11.hpp:675-679), which equals this whenever the pointer is the
// allocation's base, as in the reference's own callers; for interior pointers this check is the stricter one.
int bytes_available(const void* ptr, size_t* bytes) {
  const DriverApi& drv = driver_api();
  if (!drv.ok) return CUDA_ERROR_NOT_INITIALIZED;
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = drv.MemGetAddressRange(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *bytes = size - (reinterpret_cast<CUdeviceptr>(ptr) - base);
  return 0;
}

// One matrix check of the reference: leading dimension first, then the allocation size, with a failing
// driver query reported as an invalid buffer.
int test_matrix(size_t one, size_t two, const void* buf, size_t offset, size_t ld, size_t elem, bool test_ld,
                int bad_ld, int too_small, int invalid) {
  if (test_ld && ld < one) return bad_ld;
  if (!buf) return invalid;
  size_t have = 0;
  if (bytes_available(buf, &have) != 0) return invalid;
  const size_t required = (ld * (two - 1) + one + offset) * elem;
  if (have < required) return too_small;
  return kSuccess;
}

// Which dimension of each stored matrix is contiguous (reference: xgemm.hpp:87-107).
Extents extents(int layout, int ta, int tb, size_t m, size_t n, size_t k) {
  Extents e;
  e.a_rotated = (layout == kColMajor && ta != kNo) || (layout == kRowMajor && ta == kNo);
  e.b_rotated = (layout == kColMajor && tb != kNo) || (layout == kRowMajor && tb == kNo);
  e.c_rotated = (layout == kRowMajor);
  e.a_one = e.a_rotated ? k : m;
  e.a_two = e.a_rotated ? m : k;
  e.b_one = e.b_rotated ? n : k;
  e.b_two = e.b_rotated ? k : n;
  e.c_one = e.c_rotated ? n : m;
  e.c_two = e.c_rotated ? m : n;
  return e;
}

bool valid_enums(int layout, int ta, int tb) {
  return (layout == kRowMajor || layout == kColMajor) && (ta == kNo || ta == kYes || ta == kConjugate) &&
         (tb == kNo || tb == kYes || tb == kConjugate);
}

// Row-major problems are run as the column-major problem C^T = op(B)^T * op(A)^T on the same memory, so the
// kernels only ever see an M-contiguous C plus one "K is contiguous" bit per operand.
void normalise(GemmDesc& d, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* a, size_t a_ld,
               const void* b, size_t b_ld, void* c, size_t c_ld, const Extents& e) {
  const bool a_kc = e.a_rotated;
  const bool b_kc = !e.b_rotated;
  d.k = static_cast<long long>(k);
  d.c = c;
  d.ldc = static_cast<long long>(c_ld);
  if (layout == kColMajor) {
    d.m = static_cast<long long>(m);
    d.n = static_cast<long long>(n);
    d.a = a; d.lda = static_cast<long long>(a_ld); d.a_kcontig = a_kc; d.conj_a = (ta == kConjugate);
    d.b = b; d.ldb = static_cast<long long>(b_ld); d.b_kcontig = b_kc; d.conj_b = (tb == kConjugate);
  } else {
    d.m = static_cast<long long>(n);
    d.n = static_cast<long long>(m);
    d.a = b; d.lda = static_cast<long long>(b_ld); d.a_kcontig = b_kc; d.conj_a = (tb == kConjugate);
    d.b = a; d.ldb = static_cast<long long>(a_ld); d.b_kcontig = a_kc; d.conj_b = (ta == kConjugate);
  }
}

// ---- streams ------------------------------------------------------------------------------------------

std::mutex g_stream_mutex;
// Keyed by the context's unique id where the driver offers one: a destroyed context's handle value can be reused
// by a later context, and a stream of the dead context must not be handed out for the new one.
std::map<unsigned long long, cudaStream_t> g_streams;

// The library-owned non-blocking stream of the current context (one per context, created on first use).
int private_stream(cudaStream_t* out) {
  unsigned long long key = 0;
  const int r = context_key(&key);
  if (r != 0) return r;
  std::lock_guard<std::mutex> lock(g_stream_mutex);
  auto it = g_streams.find(key);
  if (it == g_streams.end()) {
    cudaStream_t s = nullptr;
    const cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e != cudaSuccess) return static_cast<int>(e);
    it = g_streams.emplace(key, s).first;
  }
  *out = it->second;
  return 0;
}

int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return dev;
}

// ---- dispatch -----------------------------------------------------------------------------------------

// Per-call log, off unless the environment variable B200BLAS_VERBOSE is set (the reference has a compile-time
// equivalent, -DVERBOSE: src/routines/common.cpp:69-84 prints every kernel it runs and its time). Level 1 prints one
// line per kernel launch to stderr; level 2 also waits for the kernel and prints its device time, which serialises
// the stream and is meant for debugging only.
int verbose_level() {
  static const int level = [] {
    const char* v = std::getenv("B200BLAS_VERBOSE");
    return v ? std::atoi(v) : 0;
  }();
  return level;
}

void log_launch(const GemmDesc& d, const char* name, cudaError_t err, cudaStream_t stream) {
  std::fprintf(stderr, "[b200blas] %s dtype=%d m=%lld n=%lld k=%lld batch=%lld a_kcontig=%d b_kcontig=%d tri=%d conv=%d -> %s\n",
               name, d.dtype, d.m, d.n, d.k, d.batch, d.a_kcontig, d.b_kcontig, d.tri, d.is_conv,
               err == cudaSuccess ? "enqueued" : cudaGetErrorString(err));
  if (verbose_level() > 1 && err == cudaSuccess) {
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
      cudaGetLastError();
      return;
    }
    const auto t0 = std::chrono::steady_clock::now();
    if (cudaStreamSynchronize(stream) == cudaSuccess) {
      const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
      std::fprintf(stderr, "[b200blas] %s completed, %.3f ms from launch to completion (host clock)\n", name, ms);
    }
  }
}

cudaError_t dispatch(const GemmDesc& d, cudaStream_t stream) {
  const char* name = "none";
  cudaError_t err;
  switch (d.dtype) {
    case 32:
      err = d.is_conv ? launch_tc_conv_f32(d, stream, &name) : launch_tc_f32_narrow(d, stream, &name);
      if (err == cudaErrorNotSupported && !d.is_conv) err = launch_small_batched_f32(d, stream, &name);
      if (err == cudaErrorNotSupported && !d.is_conv) err = launch_repitched(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_tc_f32_pair(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_tc_f32(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_simt_f32(d, stream, &name);
      break;
    case 64:
      err = d.is_conv ? launch_dmma_conv_f64(d, stream, &name) : launch_dmma_f64(d, stream, &name);
      if (err == cudaErrorNotSupported && d.is_conv) err = launch_conv_two_step(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_simt_f64(d, stream, &name);
      break;
    case 16:
      err = d.is_conv ? launch_tc_conv_f16(d, stream, &name) : launch_repitched(d, stream, &name);
      if (err == cudaErrorNotSupported && d.is_conv) err = launch_conv_two_step(d, stream, &name);
      if (err == cudaErrorNotSupported && !d.is_conv) err = launch_tc_f16_pair(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_tc_f16(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_simt_f16(d, stream, &name);
      break;
    case 3232:
      err = launch_complex_on_real(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_simt_c32(d, stream, &name);
      break;
    case 6464:
      err = launch_complex_on_real(d, stream, &name);
      if (err == cudaErrorNotSupported) err = launch_simt_c64(d, stream, &name);
      break;
    default: return cudaErrorInvalidValue;
  }
  t_last_kernel = name;
  if (err == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
  if (verbose_level() > 0) log_launch(d, name, err, stream);
  return err;
}

// Runs `d` either synchronously on the private stream or asynchronously on the caller's stream.
int run(const GemmDesc& d, void* stream, int async) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!async) {
    const int r = private_stream(&s);
    if (r != 0) return r;
  }
  cudaError_t err = dispatch(d, s);
  if (err == cudaSuccess && !async) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    std::fprintf(stderr, "b200blas: CUDA error %d (%s)\n", static_cast<int>(err), cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return tensor_core_status(async);
}

// After a synchronous call that ran a tensor-core kernel: the kernel reports expired waits through the status block
// (mapped host memory, so this is a plain read after the stream synchronisation the call has just done) instead of
// hanging or trapping. Asynchronous callers read it with b200blas_tensor_core_status once their stream has finished.
int tensor_core_status(int async) {
  if (!async) {
    unsigned int status[4] = {0, 0, 0, 0};
    if (tc_status_read(status, true) && status[0] != 0) {
      std::fprintf(stderr, "b200blas: tensor-core kernel gave up waiting (code %u, block %u)\n", status[0], status[1]);
      return kUnexpectedError;
    }
  }
  return kSuccess;
}

bool force_small_family(int dtype, size_t m, size_t n, size_t k) {
  const size_t t = min_indirect_size(current_device(), dtype);
  if (t == 0) return false;
  const long double lim = static_cast<long double>(t) * t * t;
  return static_cast<long double>(m) * n * k < lim;
}

int sm_budget() { return g_sm_budget.load(std::memory_order_relaxed); }

// ---- bridge for the allocation-free batched entry point ------------------------------------------------------
// Same argument checks, normalisation and table layout as b200blas_gemm_batched above, but the tables are written
// into a caller-provided host block and nothing is enqueued; the caller copies the block to its own device
// scratch, calls patch_batched_tables() with that address and launches with dispatch_desc().
int prepare_batched(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* alphas,
                    const void* a, const size_t* a_offsets, size_t a_ld, const void* b, const size_t* b_offsets,
                    size_t b_ld, const void* betas, void* c, const size_t* c_offsets, size_t c_ld, size_t batch_count,
                    unsigned char* host_block, size_t host_capacity, GemmDesc* out, BatchedTables* tables) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_enums(layout, ta, tb)) return kUnexpectedError;
  if (batch_count < 1 || !alphas || !betas || !a_offsets || !b_offsets || !c_offsets) return kInvalidBatchCount;
  if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
  const Extents e = extents(layout, ta, tb, m, n, k);
  size_t a_max = 0, b_max = 0, c_max = 0;
  for (size_t i = 0; i < batch_count; ++i) {
    if (a_offsets[i] > a_max) a_max = a_offsets[i];
    if (b_offsets[i] > b_max) b_max = b_offsets[i];
    if (c_offsets[i] > c_max) c_max = c_offsets[i];
  }
  int st = test_matrix(e.a_one, e.a_two, a, a_max, a_ld, elem, false, kInvalidLeadDimA, kInsufficientMemoryA,
                       kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(e.b_one, e.b_two, b, b_max, b_ld, elem, false, kInvalidLeadDimB, kInsufficientMemoryB,
                   kInvalidMatrixB);
  if (st) return st;
  st = test_matrix(e.c_one, e.c_two, c, c_max, c_ld, elem, true, kInvalidLeadDimC, kInsufficientMemoryC,
                   kInvalidMatrixC);
  if (st) return st;

  GemmDesc d = {};
  d.dtype = dtype;
  normalise(d, layout, ta, tb, m, n, k, a, a_ld, b, b_ld, c, c_ld, e);
  const bool swapped = (layout == kRowMajor);
  d.batch = static_cast<long long>(batch_count);
  d.force_small = force_small_family(dtype, m, n, k);

  const size_t scalar_bytes = (dtype == 16 || dtype == 32) ? 4 : (dtype == 64 || dtype == 3232) ? 8 : 16;
  const size_t off_bytes = batch_count * sizeof(long long);
  tables->off_block = (3 * off_bytes + 15) / 16 * 16;
  tables->sc_bytes = (batch_count * scalar_bytes + 15) / 16 * 16;
  tables->total = tables->off_block + 2 * tables->sc_bytes;
  tables->batch_count = batch_count;
  if (tables->total > host_capacity) return kInvalidBatchCount;
  long long* h_a = reinterpret_cast<long long*>(host_block);
  long long* h_b = h_a + batch_count;
  long long* h_c = h_b + batch_count;
  unsigned char* h_alpha = host_block + tables->off_block;
  unsigned char* h_beta = h_alpha + tables->sc_bytes;
  bool offsets_aligned = true;
  for (size_t i = 0; i < batch_count; ++i) {
    h_a[i] = static_cast<long long>(swapped ? b_offsets[i] : a_offsets[i]);
    h_b[i] = static_cast<long long>(swapped ? a_offsets[i] : b_offsets[i]);
    h_c[i] = static_cast<long long>(c_offsets[i]);
    if ((a_offsets[i] | b_offsets[i] | c_offsets[i]) & 3) offsets_aligned = false;
    double al[2], be[2];
    read_scalar(dtype, alphas, i, al);
    read_scalar(dtype, betas, i, be);
    if (dtype == 16 || dtype == 32) {
      reinterpret_cast<float*>(h_alpha)[i] = static_cast<float>(al[0]);
      reinterpret_cast<float*>(h_beta)[i] = static_cast<float>(be[0]);
    } else if (dtype == 64) {
      reinterpret_cast<double*>(h_alpha)[i] = al[0];
      reinterpret_cast<double*>(h_beta)[i] = be[0];
    } else if (dtype == 3232) {
      reinterpret_cast<float*>(h_alpha)[2 * i] = static_cast<float>(al[0]);
      reinterpret_cast<float*>(h_alpha)[2 * i + 1] = static_cast<float>(al[1]);
      reinterpret_cast<float*>(h_beta)[2 * i] = static_cast<float>(be[0]);
      reinterpret_cast<float*>(h_beta)[2 * i + 1] = static_cast<float>(be[1]);
    } else {
      reinterpret_cast<double*>(h_alpha)[2 * i] = al[0];
      reinterpret_cast<double*>(h_alpha)[2 * i + 1] = al[1];
      reinterpret_cast<double*>(h_beta)[2 * i] = be[0];
      reinterpret_cast<double*>(h_beta)[2 * i + 1] = be[1];
    }
  }
  d.tables_aligned4 = offsets_aligned ? 1 : 0;
  // Evenly spaced offsets (the common case) are also described by a first offset and a stride, which lets the
  // TMA-based kernels address the batch through one tensor map.
  const long long sa = batch_count > 1 ? h_a[1] - h_a[0] : 0;
  const long long sb = batch_count > 1 ? h_b[1] - h_b[0] : 0;
  const long long sc = batch_count > 1 ? h_c[1] - h_c[0] : 1;
  bool uniform = sa >= 0 && sb >= 0 && sc > 0;
  for (size_t i = 1; uniform && i < batch_count; ++i) {
    const long long step = static_cast<long long>(i);
    uniform = h_a[i] == h_a[0] + step * sa && h_b[i] == h_b[0] + step * sb && h_c[i] == h_c[0] + step * sc;
  }
  if (uniform) {
    d.uniform_strides = 1;
    d.a_off = h_a[0]; d.b_off = h_b[0]; d.c_off = h_c[0];
    d.a_stride = sa; d.b_stride = sb; d.c_stride = sc;
  }
  *out = d;
  return kSuccess;
}

void patch_batched_tables(GemmDesc* d, const BatchedTables& t, const unsigned char* device_block) {
  d->a_offs = reinterpret_cast<const long long*>(device_block);
  d->b_offs = d->a_offs + t.batch_count;
  d->c_offs = d->b_offs + t.batch_count;
  d->alphas = device_block + t.off_block;
  d->betas = device_block + t.off_block + t.sc_bytes;
}

cudaError_t dispatch_desc(const GemmDesc& d, cudaStream_t stream) { return dispatch(d, stream); }

int status_after_sync() { return tensor_core_status(0); }

int gemm_validate(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* a, size_t a_offset,
                  size_t a_ld, const void* b, size_t b_offset, size_t b_ld, const void* c, size_t c_offset,
                  size_t c_ld) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_enums(layout, ta, tb)) return kUnexpectedError;
  if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
  const Extents e = extents(layout, ta, tb, m, n, k);
  int st = test_matrix(e.a_one, e.a_two, a, a_offset, a_ld, elem, true, kInvalidLeadDimA, kInsufficientMemoryA,
                       kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(e.b_one, e.b_two, b, b_offset, b_ld, elem, true, kInvalidLeadDimB, kInsufficientMemoryB,
                   kInvalidMatrixB);
  if (st) return st;
  return test_matrix(e.c_one, e.c_two, c, c_offset, c_ld, elem, true, kInvalidLeadDimC, kInsufficientMemoryC,
                     kInvalidMatrixC);
}

int gemm_enqueue(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const double alpha[2],
                 const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                 const double beta[2], void* c, size_t c_offset, size_t c_ld, cudaStream_t stream, int tri,
                 int real_diag) {
  if (dtype_size(dtype) == 0 || !valid_enums(layout, ta, tb)) return kUnexpectedError;
  if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
  const Extents e = extents(layout, ta, tb, m, n, k);
  GemmDesc d = {};
  d.dtype = dtype;
  normalise(d, layout, ta, tb, m, n, k, a, a_ld, b, b_ld, c, c_ld, e);
  const bool swapped = (layout == kRowMajor);
  d.a_off = static_cast<long long>(swapped ? b_offset : a_offset);
  d.b_off = static_cast<long long>(swapped ? a_offset : b_offset);
  d.c_off = static_cast<long long>(c_offset);
  d.batch = 1;
  d.alpha[0] = alpha[0]; d.alpha[1] = alpha[1];
  d.beta[0] = beta[0]; d.beta[1] = beta[1];
  d.force_small = force_small_family(dtype, m, n, k);
  // The triangle is given for C as the caller sees it; the kernels see the normalised (column-major) C, which for a
  // row-major call is the transpose.
  d.tri = tri == 0 ? 0 : ((tri == kUpper) != swapped ? 1 : 2);
  d.real_diag = real_diag;
  const cudaError_t err = dispatch(d, stream);
  if (err != cudaSuccess) {
    std::fprintf(stderr, "b200blas: CUDA error %d (%s)\n", static_cast<int>(err), cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return kSuccess;
}

int begin_call(void* stream, int async, cudaStream_t* out) {
  *out = static_cast<cudaStream_t>(stream);
  return async ? 0 : private_stream(out);
}

int end_call(cudaStream_t stream, int async, cudaError_t err) {
  if (err == cudaSuccess && !async) err = cudaStreamSynchronize(stream);
  if (err != cudaSuccess) {
    std::fprintf(stderr, "b200blas: CUDA error %d (%s)\n", static_cast<int>(err), cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return tensor_core_status(async);
}

}  // namespace b200

using namespace b200;

extern "C" int b200blas_gemm(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* alpha,
                             const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                             const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async) {
  if (dtype_size(dtype) == 0 || !alpha || !beta) return kUnexpectedError;
  double al[2], be[2];
  read_scalar(dtype, alpha, 0, al);
  read_scalar(dtype, beta, 0, be);
  int st = gemm_validate(dtype, layout, ta, tb, m, n, k, a, a_offset, a_ld, b, b_offset, b_ld, c, c_offset, c_ld);
  if (st != kSuccess) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  st = gemm_enqueue(dtype, layout, ta, tb, m, n, k, al, a, a_offset, a_ld, b, b_offset, b_ld, be, c, c_offset, c_ld, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_gemm_strided_batched(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k,
                                             const void* alpha, const void* a, size_t a_offset, size_t a_ld,
                                             size_t a_stride, const void* b, size_t b_offset, size_t b_ld,
                                             size_t b_stride, const void* beta, void* c, size_t c_offset, size_t c_ld,
                                             size_t c_stride, size_t batch_count, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_enums(layout, ta, tb) || !alpha || !beta) return kUnexpectedError;
  if (batch_count < 1) return kInvalidBatchCount;
  if (c_stride == 0) return kInvalidDimension;
  if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
  const Extents e = extents(layout, ta, tb, m, n, k);
  const size_t last = batch_count - 1;
  int st = test_matrix(e.a_one, e.a_two, a, a_offset + last * a_stride, a_ld, elem, true, kInvalidLeadDimA,
                       kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(e.b_one, e.b_two, b, b_offset + last * b_stride, b_ld, elem, true, kInvalidLeadDimB,
                   kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  st = test_matrix(e.c_one, e.c_two, c, c_offset + last * c_stride, c_ld, elem, true, kInvalidLeadDimC,
                   kInsufficientMemoryC, kInvalidMatrixC);
  if (st) return st;

  GemmDesc d = {};
  d.dtype = dtype;
  normalise(d, layout, ta, tb, m, n, k, a, a_ld, b, b_ld, c, c_ld, e);
  const bool swapped = (layout == kRowMajor);
  d.a_off = static_cast<long long>(swapped ? b_offset : a_offset);
  d.b_off = static_cast<long long>(swapped ? a_offset : b_offset);
  d.c_off = static_cast<long long>(c_offset);
  d.a_stride = static_cast<long long>(swapped ? b_stride : a_stride);
  d.b_stride = static_cast<long long>(swapped ? a_stride : b_stride);
  d.c_stride = static_cast<long long>(c_stride);
  d.batch = static_cast<long long>(batch_count);
  read_scalar(dtype, alpha, 0, d.alpha);
  read_scalar(dtype, beta, 0, d.beta);
  d.force_small = force_small_family(dtype, m, n, k);
  return run(d, stream, async);
}

extern "C" int b200blas_gemm_batched(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k,
                                     const void* alphas, const void* a, const size_t* a_offsets, size_t a_ld,
                                     const void* b, const size_t* b_offsets, size_t b_ld, const void* betas, void* c,
                                     const size_t* c_offsets, size_t c_ld, size_t batch_count, void* stream,
                                     int async) {
  // Argument checks, normalisation and the per-batch tables (three offset tables, then alphas and betas converted
  // to the kernel's compute type) are shared with the allocation-free entry point. As in the reference, the
  // leading dimensions of A and B are deliberately not tested for this routine.
  if (batch_count < 1 || batch_count > kMaxBatchCount || !alphas || !betas || !a_offsets || !b_offsets || !c_offsets)
    return kInvalidBatchCount;
  std::vector<unsigned char> host;
  try {
    host.resize(3 * sizeof(long long) * batch_count + 16 + 2 * (16 * batch_count + 16));
  } catch (...) {
    return kUnexpectedError;
  }
  GemmDesc d = {};
  BatchedTables tables = {};
  const int st = prepare_batched(dtype, layout, ta, tb, m, n, k, alphas, a, a_offsets, a_ld, b, b_offsets, b_ld, betas,
                                 c, c_offsets, c_ld, batch_count, host.data(), host.size(), &d, &tables);
  if (st != kSuccess) return st;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!async) {
    const int r = private_stream(&s);
    if (r != 0) return r;
  }
  // Stream-ordered scratch: allocated, filled, used and released in stream order, so concurrent calls on
  // different streams never share it. The host block is pageable, so the copy has left it when the call returns.
  unsigned char* dev = nullptr;
  cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&dev), tables.total, s);
  if (err == cudaSuccess) err = cudaMemcpyAsync(dev, host.data(), tables.total, cudaMemcpyHostToDevice, s);
  if (err == cudaSuccess) {
    patch_batched_tables(&d, tables, dev);
    err = dispatch(d, s);
  }
  if (dev) {
    const cudaError_t ferr = cudaFreeAsync(dev, s);
    if (err == cudaSuccess) err = ferr;
  }
  if (err == cudaSuccess && !async) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    std::fprintf(stderr, "b200blas: CUDA error %d (%s)\n", static_cast<int>(err), cudaGetErrorString(err));
    return static_cast<int>(err);
  }
  return tensor_core_status(async);
}

extern "C" int b200blas_convgemm(int dtype, int kernel_mode, size_t channels, size_t height, size_t width,
                                 size_t kernel_h, size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h,
                                 size_t stride_w, size_t dilation_h, size_t dilation_w, size_t num_kernels,
                                 size_t batch_count, const void* im, size_t im_offset, const void* kernel,
                                 size_t kernel_offset, void* result, size_t result_offset, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || dtype > 64) return kNotImplemented;
  if (kernel_mode != kCrossCorrelation && kernel_mode != kConvolution) return kUnexpectedError;
  if (batch_count == 0) return kInvalidBatchCount;
  if (channels == 0 || height == 0 || width == 0 || num_kernels == 0) return kInvalidDimension;
  if (kernel_h == 0 || kernel_w == 0 || stride_h == 0 || stride_w == 0) return kInvalidDimension;
  // Output extents; a dilated kernel larger than the padded image yields extent 1, as in the reference
  // (src/routines/levelx/xconvgemm.cpp:67-72).
  const size_t size_h = height + 2 * pad_h;
  const size_t padding_h = dilation_h * (kernel_h - 1) + 1;
  const size_t output_h = (size_h >= padding_h) ? (size_h - padding_h) / stride_h + 1 : 1;
  const size_t size_w = width + 2 * pad_w;
  const size_t padding_w = dilation_w * (kernel_w - 1) + 1;
  const size_t output_w = (size_w >= padding_w) ? (size_w - padding_w) / stride_w + 1 : 1;
  const size_t patch_size = kernel_h * kernel_w * channels;
  const size_t num_patches = output_h * output_w;
  const size_t result_stride = num_kernels * num_patches;

  int st = test_matrix(patch_size, num_kernels, kernel, kernel_offset, patch_size, elem, true, kInvalidLeadDimB,
                       kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  st = test_matrix(num_patches, num_kernels, result, result_offset + result_stride * (batch_count - 1), num_patches,
                   elem, true, kInvalidLeadDimC, kInsufficientMemoryC, kInvalidMatrixC);
  if (st) return st;
  if (!im) return kInvalidMatrixA;
  const size_t int_max = 0x7FFFFFFF;
  if (channels * height * width > int_max || patch_size > int_max || num_patches > int_max) return kInvalidDimension;

  GemmDesc d = {};
  d.dtype = dtype;
  d.is_conv = 1;
  d.m = static_cast<long long>(num_patches);
  d.n = static_cast<long long>(num_kernels);
  d.k = static_cast<long long>(patch_size);
  d.a = im;
  d.a_off = static_cast<long long>(im_offset);
  d.a_stride = static_cast<long long>(channels * height * width);
  d.lda = 0;
  d.b = kernel;
  d.b_off = static_cast<long long>(kernel_offset);
  d.ldb = static_cast<long long>(patch_size);
  d.b_kcontig = 1;
  d.b_stride = 0;
  d.c = result;
  d.c_off = static_cast<long long>(result_offset);
  d.ldc = static_cast<long long>(num_patches);
  d.c_stride = static_cast<long long>(result_stride);
  d.batch = static_cast<long long>(batch_count);
  d.alpha[0] = 1.0;
  d.beta[0] = 0.0;
  d.conv.channels = static_cast<int>(channels);
  d.conv.height = static_cast<int>(height);
  d.conv.width = static_cast<int>(width);
  d.conv.kernel_h = static_cast<int>(kernel_h);
  d.conv.kernel_w = static_cast<int>(kernel_w);
  d.conv.pad_h = static_cast<int>(pad_h);
  d.conv.pad_w = static_cast<int>(pad_w);
  d.conv.stride_h = static_cast<int>(stride_h);
  d.conv.stride_w = static_cast<int>(stride_w);
  d.conv.dil_h = static_cast<int>(dilation_h);
  d.conv.dil_w = static_cast<int>(dilation_w);
  d.conv.out_w = static_cast<int>(output_w);
  d.conv.flip = (kernel_mode == kConvolution);
  return run(d, stream, async);
}

extern "C" int b200blas_gemm_temp_buffer_size(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k,
                                              size_t, size_t, size_t, size_t, size_t, size_t,
                                              size_t* temp_buffer_size) {
  if (dtype_size(dtype) == 0 || !valid_enums(layout, ta, tb) || !temp_buffer_size) return kUnexpectedError;
  if (m == 0 || n == 0 || k == 0) return kInvalidDimension;
  *temp_buffer_size = 0;
  return kSuccess;
}

extern "C" void b200blas_set_sm_budget(int sms) { g_sm_budget.store(sms > 0 ? sms : 0, std::memory_order_relaxed); }

extern "C" int b200blas_clear_cache(void) { return kSuccess; }
extern "C" int b200blas_fill_cache(int) { return kSuccess; }

extern "C" int b200blas_tensor_core_status(unsigned int out[4], int clear) {
  unsigned int status[4] = {0, 0, 0, 0};
  if (!tc_status_read(status, clear != 0)) return kUnexpectedError;
  if (out) std::memcpy(out, status, sizeof(status));
  return status[0] != 0 ? kUnexpectedError : kSuccess;
}

extern "C" const char* b200blas_last_kernel(void) { return t_last_kernel; }
extern "C" uint64_t b200blas_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" const char* b200blas_version(void) { return "b200blas 0.1 (sm_100a)"; }
