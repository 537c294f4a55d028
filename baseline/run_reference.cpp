// Times the reference library's own CUDA build on the current GPU: the same calls, shapes and data distributions as
// bench.py's sweep, through the reference's public API (include/clblast_cuda.h), and prints one JSON object.
//
// Convention of the reference's own client (test/performance/client.cpp:419-468): wall clock around the
// host-synchronous call, minimum (and here also median) over the runs, after warm-up calls that absorb the run-time
// compilation of the kernels. Only single and double precision: the reference's CUDA flavour cannot compile half.
#include <cuda.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <algorithm>
#include <cstring>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include <clblast_cuda.h>

// The reference hands NVRTC the OpenCL option "-cl-std=CL1.1" (src/utilities/utilities.cpp:673-682 is called for the
// CUDA flavour too, src/routine.cpp:107), which NVRTC rejects with NVRTC_ERROR_INVALID_OPTION, so its CUDA flavour
// cannot compile any kernel as it stands. Unless REFERENCE_STOCK_OPTIONS is set, this program interposes
// nvrtcCompileProgram and drops the options that start with "-cl-"; nothing else of the reference is touched. The JSON
// says which of the two was measured.
static bool g_filter_options = true;
static int g_dropped_options = 0;

extern "C" nvrtcResult nvrtcCompileProgram(nvrtcProgram prog, int num_options, const char* const* options) {
  using Fn = nvrtcResult (*)(nvrtcProgram, int, const char* const*);
  static Fn real = reinterpret_cast<Fn>(dlsym(RTLD_NEXT, "nvrtcCompileProgram"));
  if (!real) return NVRTC_ERROR_INTERNAL_ERROR;
  std::vector<const char*> kept;
  for (int i = 0; i < num_options; ++i) {
    if (g_filter_options && std::strncmp(options[i], "-cl-", 4) == 0) {
      ++g_dropped_options;
      continue;
    }
    kept.push_back(options[i]);
  }
  return real(prog, static_cast<int>(kept.size()), kept.data());
}

namespace {

#define CHECK_CU(call)                                                          \
  do {                                                                          \
    const CUresult r_ = (call);                                                 \
    if (r_ != CUDA_SUCCESS) {                                                   \
      std::printf("{\"unavailable\": \"%s failed with %d\"}\n", #call, (int)r_); \
      return 0;                                                                 \
    }                                                                           \
  } while (0)

template <typename T>
CUdeviceptr upload_uniform(size_t count, unsigned seed, double lo, double hi) {
  std::vector<T> host(count);
  std::mt19937 gen(seed);
  std::uniform_real_distribution<double> dist(lo, hi);
  for (auto& v : host) v = static_cast<T>(dist(gen));
  CUdeviceptr d = 0;
  if (cuMemAlloc(&d, count * sizeof(T)) != CUDA_SUCCESS) return 0;
  cuMemcpyHtoD(d, host.data(), count * sizeof(T));
  return d;
}

struct Timing {
  double min_ms, median_ms;
  int status;
};

template <typename F>
Timing time_call(F&& call, int warmup, int runs) {
  Timing t = {0.0, 0.0, 0};
  for (int i = 0; i < warmup; ++i) {
    t.status = static_cast<int>(call());
    if (t.status != 0) return t;
  }
  std::vector<double> ms;
  for (int i = 0; i < runs; ++i) {
    const auto t0 = std::chrono::steady_clock::now();
    t.status = static_cast<int>(call());
    const auto t1 = std::chrono::steady_clock::now();
    if (t.status != 0) return t;
    ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
  }
  std::sort(ms.begin(), ms.end());
  t.min_ms = ms.front();
  t.median_ms = ms[ms.size() / 2];
  return t;
}

void report(const char* name, const Timing& t, double flops, bool last = false) {
  if (t.status != 0) {
    std::printf("\"%s\": {\"status\": %d}%s", name, t.status, last ? "" : ", ");
  } else {
    std::printf("\"%s\": {\"min_ms\": %.5f, \"median_ms\": %.5f, \"tflops\": %.4f, \"tflops_median\": %.4f}%s", name,
                t.min_ms, t.median_ms, flops / (t.min_ms * 1e-3) / 1e12, flops / (t.median_ms * 1e-3) / 1e12,
                last ? "" : ", ");
  }
  std::fflush(stdout);
}

template <typename T>
Timing gemm_case(clblast::Layout layout, size_t m, size_t n, size_t k, T alpha, T beta, size_t ld_pad, CUcontext ctx,
                 CUdevice dev, int runs) {
  const bool row = layout == clblast::Layout::kRowMajor;
  const size_t a_ld = (row ? k : m) + ld_pad, b_ld = (row ? n : k) + ld_pad, c_ld = (row ? n : m) + ld_pad;
  const CUdeviceptr a = upload_uniform<T>(a_ld * (row ? m : k), 1, -1, 1);
  const CUdeviceptr b = upload_uniform<T>(b_ld * (row ? k : n), 2, -1, 1);
  const CUdeviceptr c = upload_uniform<T>(c_ld * (row ? m : n), 3, -1, 1);
  Timing t = {0, 0, -1};
  if (a && b && c) {
    t = time_call([&] {
      return clblast::Gemm<T>(layout, clblast::Transpose::kNo, clblast::Transpose::kNo, m, n, k, alpha, a, 0, a_ld, b, 0,
                              b_ld, beta, c, 0, c_ld, ctx, dev);
    }, 2, runs);
  }
  cuMemFree(a); cuMemFree(b); cuMemFree(c);
  return t;
}

}  // namespace

int main() {
  CHECK_CU(cuInit(0));
  CUdevice dev;
  CHECK_CU(cuDeviceGet(&dev, 0));
  CUcontext ctx;
  CHECK_CU(cuDevicePrimaryCtxRetain(&ctx, dev));
  CHECK_CU(cuCtxSetCurrent(ctx));
  using clblast::Layout;
  g_filter_options = std::getenv("REFERENCE_STOCK_OPTIONS") == nullptr;
  std::printf("{\"how\": \"the reference's CUDA build (kernels compiled at run time by NVRTC), wall clock around the "
              "host-synchronous call, 2 warm-up calls, min and median of the runs\", \"nvrtc_options\": \"%s\", ",
              g_filter_options ? "the reference's options minus '-cl-std=CL1.1', which NVRTC rejects (status -2040 with the stock options)"
                               : "stock");
  report("sgemm_1024", gemm_case<float>(Layout::kRowMajor, 1024, 1024, 1024, 0.7f, 0.3f, 0, ctx, dev, 20), 2.0 * 1024 * 1024 * 1024);
  report("sgemm_1000", gemm_case<float>(Layout::kColMajor, 1000, 1000, 1000, 1.5f, 0.5f, 16, ctx, dev, 20), 2.0 * 1000 * 1000 * 1000);
  report("sgemm_2048", gemm_case<float>(Layout::kColMajor, 2048, 2048, 2048, 1.5f, 0.5f, 16, ctx, dev, 10), 2.0 * 2048 * 2048 * 2048);
  report("sgemm_4096", gemm_case<float>(Layout::kColMajor, 4096, 4096, 4096, 1.5f, 0.5f, 16, ctx, dev, 10), 2.0 * 4096 * 4096 * 4096);
  report("sgemm_ragged", gemm_case<float>(Layout::kColMajor, 4097, 3071, 1025, 1.5f, 0.5f, 16, ctx, dev, 10), 2.0 * 4097 * 3071 * 1025);
  report("sgemm_8192", gemm_case<float>(Layout::kColMajor, 8192, 8192, 8192, 1.5f, 0.5f, 16, ctx, dev, 5), 2.0 * 8192 * 8192 * 8192);
  report("dgemm_8192", gemm_case<double>(Layout::kColMajor, 8192, 8192, 8192, 1.0, 0.0, 0, ctx, dev, 3), 2.0 * 8192 * 8192 * 8192);
  {  // strided batches of small problems
    const size_t batch = 8192, s = 32 * 32;
    const CUdeviceptr a = upload_uniform<float>(batch * s, 4, -1, 1), b = upload_uniform<float>(batch * s, 5, -1, 1),
                      c = upload_uniform<float>(batch * s, 6, -1, 1);
    report("batched_32", time_call([&] {
      return clblast::GemmStridedBatched<float>(Layout::kColMajor, clblast::Transpose::kNo, clblast::Transpose::kNo, 32, 32,
                                                32, 1.0f, a, 0, 32, s, b, 0, 32, s, 1.0f, c, 0, 32, s, batch, ctx, dev);
    }, 2, 20), 2.0 * 32 * 32 * 32 * batch);
    cuMemFree(a); cuMemFree(b); cuMemFree(c);
  }
  {
    const size_t batch = 2048, m = 64, n = 128, k = 96;
    const CUdeviceptr a = upload_uniform<float>(batch * m * k, 7, -1, 1), b = upload_uniform<float>(batch * k * n, 8, -1, 1),
                      c = upload_uniform<float>(batch * m * n, 9, -1, 1);
    report("batched_64x128x96", time_call([&] {
      return clblast::GemmStridedBatched<float>(Layout::kColMajor, clblast::Transpose::kNo, clblast::Transpose::kNo, m, n, k,
                                                1.0f, a, 0, m, m * k, b, 0, k, k * n, 1.0f, c, 0, m, m * n, batch, ctx, dev);
    }, 2, 20), 2.0 * m * n * k * batch);
    cuMemFree(a); cuMemFree(b); cuMemFree(c);
  }
  {  // the 56 x 56 convolution
    const size_t batch = 32, ch = 64, hw = 56, nk = 128;
    const CUdeviceptr im = upload_uniform<float>(batch * ch * hw * hw, 10, -1, 1), ker = upload_uniform<float>(nk * ch * 9, 11, -0.1, 0.1),
                      res = upload_uniform<float>(batch * nk * hw * hw, 12, 0, 0);
    report("conv_56", time_call([&] {
      return clblast::Convgemm<float>(clblast::KernelMode::kCrossCorrelation, ch, hw, hw, 3, 3, 1, 1, 1, 1, 1, 1, nk, batch,
                                      im, 0, ker, 0, res, 0, ctx, dev);
    }, 2, 10), 2.0 * batch * hw * hw * nk * ch * 9, true);
    cuMemFree(im); cuMemFree(ker); cuMemFree(res);
  }
  std::printf("}\n");
  cuDevicePrimaryCtxRelease(dev);
  return 0;
}
