// Half-precision Convgemm as an implicit GEMM on tcgen05 (kind::f16, fp32 accumulation in TMEM) with op(A), the
// im2col matrix, in tensor memory only.
//
// Replaces, for large half-precision convolutions, the reference's XconvgemmNormal / XconvgemmFlip kernels
// (src/kernels/levelx/xconvgemm_part1.opencl:22-113, xconvgemm_part2.opencl:27-336, launched from
// src/routines/levelx/xconvgemm.cpp:50-161) and its im2col + GEMM alternative (xconvgemm.cpp:96-112). Per image the
// product is result[co][pixel] = sum_k weights[co][k] * image[c(k)][h(pixel) + dh(k)][w(pixel) + dw(k)], k = (c, kh, kw)
// with kw fastest, zero outside the image, taps mirrored for kConvolution.
//
// One CTA per 128 pixels x 128 filters, persistent over (pixel tile, filter tile, image). 512 threads:
//   warp 0      TMA producer: weights [Cout][K], K-major, 64 halves = one 128-byte swizzle row per filter and K block
//   warp 1      owns TMEM, one lane issues tcgen05.mma.kind::f16 with A from tensor memory
//   warps 4-11  gather: a thread owns one output pixel (= one TMEM lane). Two groups of four warps take alternate K
//               blocks; a thread loads the 64 taps of its pixel for the group's next K block (consecutive lanes are
//               consecutive pixels, so a load instruction reads one contiguous run), packs them in pairs and writes 32
//               columns with tcgen05.st. What a K row means (channel plane, tap row and column) is decoded once per
//               launch into a table in shared memory.
//   warp 2      asks L2 for the image rows of the tile after next (cp.async.bulk.prefetch.L2, one contiguous run per
//               channel), so that the gather of a tile never waits for HBM
//   warps 12-15 epilogue: tcgen05.ld of the finished accumulator (two of them alternate, so the next tile's MMAs run
//               meanwhile), rounding to half, stores along the pixels (contiguous in the result).
// TMEM columns: [0, 256) two accumulators, [256, 384) four slots of 32 columns for op(A).
// All waits are bounded; on expiry a code is left in the status block and the CTA drains and exits.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>

#include "../runtime_state.h"
#include "../tc_host.h"
#include "launchers.h"
#include "level3_aux.h"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int BM = 128;   // output pixels per tile
constexpr int BN = 128;   // filters per tile
constexpr int BK = 64;    // halves per K block = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;        // weight tiles in flight
constexpr int A_SLOTS = 4;       // op(A) K blocks in tensor memory
constexpr int B_BYTES = BN * BK * 2;
constexpr int TMEM_COLS = 512;
constexpr int A_COL0 = 2 * BN;   // first column of the op(A) slots
constexpr int NUM_THREADS = 512;
constexpr int SMEM_FIXED = STAGES * B_BYTES + 1024 + 512;  // + 8 bytes per K row of the padded K extent

struct HalfConvParams {
  unsigned int* status;
  const __half* image;
  __half* result;
  long long image_stride, result_stride;  // elements between consecutive images
  int m, n, k;                            // pixels per image, filters, channels * taps
  int tiles_m, tiles_n, k_blocks, batch;
  ConvGeom conv;
};

__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_st_8cols(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
hconv_tc_kernel(const __grid_constant__ CUtensorMap map_b, const HalfConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * B_BYTES);
  const uint32_t bar_base = smem_u32(bars);
  // [0,S) weights landed, [S,2S) stage free, then A slot full x4, A slot free x4, accumulator full x2, empty x2
  auto b_full = [&](int s) { return bar_base + 8u * s; };
  auto b_free = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto a_full = [&](int l) { return bar_base + 8u * (2 * STAGES + l); };
  auto a_free = [&](int l) { return bar_base + 8u * (2 * STAGES + A_SLOTS + l); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 * A_SLOTS + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 * A_SLOTS + 2 + a); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * A_SLOTS + 4);
  static_assert((2 * STAGES + 2 * A_SLOTS + 4) * 8 + 12 <= 512, "barrier block");
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* const tiles_started = abort_flag + 1;  // written by the MMA lane, read by the prefetch warp
  // one entry per K row of the padded K extent: {offset of the tap from the pixel's own offset, (kh * dilation) << 16 |
  // kw * dilation}; rows beyond K get a tap row that is outside every image
  int2* const tap_table = reinterpret_cast<int2*>(reinterpret_cast<uint8_t*>(bars) + 512);

  // broadcast from lane 0: the compiler then knows the value is the same for the whole warp
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n * p.batch;
  auto tile_coords = [&](int tile, int& tm, int& tn, int& image) {  // pixels fastest, then filters, then images
    tm = tile % p.tiles_m;
    const int rest = tile / p.tiles_m;
    tn = rest % p.tiles_n;
    image = rest / p.tiles_n;
  };

  {
    const int khw = p.conv.kernel_h * p.conv.kernel_w;
    for (int kg = threadIdx.x; kg < p.k_blocks * BK; kg += NUM_THREADS) {
      int2 e = make_int2(0, 0x7FFF0000);
      if (kg < p.k) {
        const int c_id = kg / khw;
        const int k2 = kg - c_id * khw;
        int kh_id = k2 / p.conv.kernel_w;
        int kw_id = k2 - kh_id * p.conv.kernel_w;
        if (p.conv.flip) {
          kh_id = p.conv.kernel_h - 1 - kh_id;
          kw_id = p.conv.kernel_w - 1 - kw_id;
        }
        const int dh = kh_id * p.conv.dil_h, dw = kw_id * p.conv.dil_w;
        e.x = (c_id * p.conv.height + dh) * p.conv.width + dw;
        e.y = (dh << 16) | dw;
      }
      tap_table[kg] = e;
    }
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(b_full(s), 1);
      mbar_init(b_free(s), 1);
    }
    for (int l = 0; l < A_SLOTS; ++l) {
      mbar_init(a_full(l), 4);  // one arrival per warp of the group that fills the slot
      mbar_init(a_free(l), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full(a), 1);
      mbar_init(acc_empty(a), 4);
    }
    *abort_flag = 0;
    *tiles_started = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: the weight tile of every K block ----
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn, image;
        tile_coords(tile, tm, tn, image);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(b_free(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(b_full(stage), B_BYTES);
          tma_load_3d(tiles_base + stage * B_BYTES, &map_b, b_full(stage), kb * BK, tn * BN, 0);
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {  // let the copies in flight land before the CTA leaves
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long start = clock64();
          int s = stage - 1 - i;
          if (s < 0) s += STAGES;
          const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          while (!mbar_try_wait(b_full(s), par) && clock64() - start < kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: A (128 pixels x 16 k = 8 columns) from tensor memory, B from shared memory ----
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0, 0);
      int stage = 0, slot = 0, local = 0;
      uint32_t phase = 0, slot_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        *tiles_started = local + 1;
        if (!mbar_wait(acc_empty(acc), (static_cast<uint32_t>(local >> 1) & 1u) ^ 1u, abort_flag, 2u, p.status)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(b_full(stage), phase, abort_flag, 3u, p.status)) { ok = false; break; }
          if (!mbar_wait(a_full(slot), slot_phase, abort_flag, 4u, p.status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t db = smem_desc(tiles_base + stage * B_BYTES, 16, 1024, kLayoutSw128);
          const uint32_t a_tmem = tmem_base + static_cast<uint32_t>(A_COL0 + 32 * slot);
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks)
            umma_f16_ts(d_tmem, a_tmem + 8u * ks, db + 2u * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
          umma_commit(b_free(stage));
          umma_commit(a_free(slot));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if (++slot == A_SLOTS) { slot = 0; slot_phase ^= 1u; }
        }
        if (ok) umma_commit(acc_full(acc));
      }
    }
  } else if (warp == 2) {
    // ---- L2 prefetch of the image rows a tile's taps touch: per channel one contiguous run of input rows ----
    const unsigned short* const image_all = reinterpret_cast<const unsigned short*>(p.image);
    auto prefetch_tile = [&](int tile) {
      int tm, tn, image;
      tile_coords(tile, tm, tn, image);
      if (tn != 0) return;  // the filter tiles of one pixel tile read the same rows
      const int first_pixel = tm * BM;
      const int last_pixel = min(first_pixel + BM, p.m) - 1;
      int h_lo = (first_pixel / p.conv.out_w) * p.conv.stride_h - p.conv.pad_h;
      int h_hi = (last_pixel / p.conv.out_w) * p.conv.stride_h - p.conv.pad_h + (p.conv.kernel_h - 1) * p.conv.dil_h;
      h_lo = max(h_lo, 0);
      h_hi = min(h_hi, p.conv.height - 1);
      if (h_hi < h_lo) return;
      const unsigned short* const base = image_all + image * p.image_stride;
      for (int c = lane; c < p.conv.channels; c += 32) {
        // whole 16-byte granules that contain bytes of the run: inside the pages the run itself lies in
        const uintptr_t begin = reinterpret_cast<uintptr_t>(base + (static_cast<long long>(c) * p.conv.height + h_lo) * p.conv.width);
        const uintptr_t end = reinterpret_cast<uintptr_t>(base + (static_cast<long long>(c) * p.conv.height + h_hi + 1) * p.conv.width);
        const uintptr_t from = begin & ~static_cast<uintptr_t>(15);
        const uint32_t bytes = static_cast<uint32_t>(((end + 15) & ~static_cast<uintptr_t>(15)) - from);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(from), "r"(bytes) : "memory");
      }
    };
    int local = 0;
    if (static_cast<int>(blockIdx.x) < num_tiles) prefetch_tile(blockIdx.x);
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      // Two tiles ahead of the MMAs at most. A plain counter, not an mbarrier: this warp may fall behind without
      // harm, and a phase bit it has missed twice would look like one it still has to wait for. Prefetching is
      // optional, so the warp just stops when the bounded wait runs out or another role has given up.
      const long long start = clock64();
      bool go = true;
      while (*tiles_started < local) {
        __nanosleep(200);
        if (*abort_flag || clock64() - start > kWaitCycles) { go = false; break; }
      }
      if (!__all_sync(0xffffffffu, go)) break;
      if (tile + static_cast<int>(gridDim.x) < num_tiles) prefetch_tile(tile + gridDim.x);
    }
  } else if (warp >= 12) {
    // ---- epilogue: warp w reads TMEM lanes [32 (w % 4), +32) = 32 consecutive pixels, all 128 filters ----
    const int quad = warp & 3;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int tm, tn, image;
      tile_coords(tile, tm, tn, image);
      const int acc = local & 1;
      ok = mbar_wait(acc_full(acc), static_cast<uint32_t>(local >> 1) & 1u, abort_flag, 5u, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const int pixel = tm * BM + quad * 32 + lane;
      __half* const out = p.result + image * p.result_stride + pixel;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll
      for (int cb = 0; cb < BN / 32; ++cb) {
        uint32_t r[32];
        tmem_ld_32cols(t_row + cb * 32, r);
        if (pixel < p.m) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int co = tn * BN + cb * 32 + j;
            if (co < p.n) out[static_cast<long long>(co) * p.m] = __float2half_rn(__uint_as_float(r[j]));
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(acc));
    }
  } else if (warp >= 4) {
    // ---- gather: warps 4..11, two groups of four (one warp per TMEM lane quadrant each) on alternate K blocks ----
    const int quad = warp & 3;
    const int group = (warp - 4) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const unsigned short* const image_all = reinterpret_cast<const unsigned short*>(p.image);
    uint32_t g[32];  // 64 taps of this thread's pixel, two per register (lower k in the lower half)
    // where the gather stands: tile, K block, and what depends on the tile's pixel
    int g_tile = blockIdx.x, g_kb = group;
    const unsigned short* g_image = nullptr;
    int g_h0 = 0, g_w0 = 0, g_off = 0;
    auto enter_tile = [&]() {
      int tm, tn, image;
      tile_coords(g_tile, tm, tn, image);
      g_image = image_all + image * p.image_stride;
      const int pixel = tm * BM + row_in_tile;
      const int ho = pixel / p.conv.out_w, wo = pixel - ho * p.conv.out_w;
      const int h_first = ho * p.conv.stride_h - p.conv.pad_h;
      g_w0 = wo * p.conv.stride_w - p.conv.pad_w;
      g_off = h_first * p.conv.width + g_w0;
      g_h0 = pixel < p.m ? h_first : -0x20000000;  // pixels beyond the image: a row no tap can bring back inside
    };
    auto gather = [&]() {
      const int2* const taps = tap_table + g_kb * BK;
#pragma unroll
      for (int j0 = 0; j0 < 64; j0 += 8) {
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int2 e = taps[j0 + j];  // the same address for every lane: one broadcast read
          const bool inside = static_cast<unsigned>(g_h0 + (e.y >> 16)) < static_cast<unsigned>(p.conv.height) &&
                              static_cast<unsigned>(g_w0 + (e.y & 0xFFFF)) < static_cast<unsigned>(p.conv.width);
          v[j] = inside ? static_cast<uint32_t>(g_image[e.x + g_off]) : 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) g[(j0 >> 1) + j] = v[2 * j] | (v[2 * j + 1] << 16);
        asm volatile("" ::: "memory");  // eight taps at a time keep the register need bounded
      }
    };
    auto advance = [&]() {  // the group's next K block: two further in the CTA's running order
      g_kb += 2;
      bool moved = false;
      while (g_kb >= p.k_blocks && g_tile < num_tiles) {
        g_kb -= p.k_blocks;
        g_tile += gridDim.x;
        moved = true;
      }
      if (moved && g_tile < num_tiles) enter_tile();
    };
    while (g_kb >= p.k_blocks && g_tile < num_tiles) {  // a tile of one K block: group 1 starts in the next tile
      g_kb -= p.k_blocks;
      g_tile += gridDim.x;
    }
    if (g_tile < num_tiles) {
      enter_tile();
      gather();
    }
    bool ok = true;
    int kbg = 0;  // running K-block count of this CTA
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < p.k_blocks; ++kb, ++kbg) {
        if ((kbg & 1) != group) continue;
        const int slot = kbg % A_SLOTS;
        ok = mbar_wait(a_free(slot), (static_cast<uint32_t>(kbg / A_SLOTS) & 1u) ^ 1u, abort_flag, 6u, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t col0 = lane_base + static_cast<uint32_t>(A_COL0 + 32 * slot);
#pragma unroll
        for (int b8 = 0; b8 < 4; ++b8) {
          uint32_t x[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] = g[b8 * 8 + i];
          tmem_st_8cols(col0 + 8u * b8, x);
        }
        advance();
        if (g_tile < num_tiles) gather();  // in flight while the stores complete and the MMAs run
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(slot));
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace

cudaError_t launch_tc_conv_f16(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 16 || !d.is_conv || d.force_small) return cudaErrorNotSupported;
  static const bool disabled = [] {  // B200BLAS_CONV=simt | im2col: the CUDA-core kernel / the two-step route
    const char* v = std::getenv("B200BLAS_CONV");
    return v != nullptr && (std::strcmp(v, "simt") == 0 || std::strcmp(v, "im2col") == 0);
  }();
  if (disabled) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF || d.batch > 0x7FFFFFFF) return cudaErrorNotSupported;
  const long long tiles_m = (d.m + BM - 1) / BM, tiles_n = (d.n + BN - 1) / BN;
  const long long tiles = tiles_m * tiles_n * d.batch;
  if (d.m < 128 || d.n < 32 || d.k < 64 || tiles < 64 || tiles > 0x7FFFFFFF) return cudaErrorNotSupported;
  // 32-bit offsets inside an image, 16-bit tap offsets, and the tap table must fit beside the weight ring
  const long long image_span = (static_cast<long long>(d.conv.channels) * d.conv.height +
                                static_cast<long long>(d.conv.kernel_h) * d.conv.dil_h + d.conv.pad_h + d.conv.stride_h) *
                                   d.conv.width + static_cast<long long>(d.conv.kernel_w) * d.conv.dil_w;
  const bool taps_fit = d.conv.height < 0x7000 && d.conv.width < 0x7000 && d.conv.pad_h < 0x800 &&
                        static_cast<long long>(d.conv.kernel_h) * d.conv.dil_h < 0x7000 &&
                        static_cast<long long>(d.conv.kernel_w) * d.conv.dil_w < 0x7000;
  const long long k_blocks = (d.k + BK - 1) / BK;
  const long long smem = SMEM_FIXED + 8 * k_blocks * BK;
  if (!taps_fit || image_span >= 0x20000000LL || smem > 227 * 1024) return cudaErrorNotSupported;

  // Weights [Cout][K] travel by TMA: a base that is not 16-byte aligned or a K that is not a multiple of 8 halves is
  // copied once into scratch with an aligned pitch.
  const __half* weights = static_cast<const __half*>(d.b) + d.b_off;
  long long pitch = d.ldb;
  __half* scratch = nullptr;
  struct Release {
    __half*& ptr; cudaStream_t stream;
    ~Release() { if (ptr) cudaFreeAsync(ptr, stream); }
  } release{scratch, stream};
  if ((reinterpret_cast<uintptr_t>(weights) & 15) || (d.ldb % 8)) {
    pitch = (d.k + 7) / 8 * 8;
    cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&scratch), static_cast<size_t>(d.n) * pitch * 2, stream);
    if (err != cudaSuccess) return err;
    RepitchJob jobs[2] = {};
    jobs[0] = {weights, scratch, d.k, d.n, d.ldb, pitch};
    err = launch_repitch(2, jobs, stream);
    if (err != cudaSuccess) return err;
    weights = scratch;
  }
  CUtensorMap map_b;
  if (!encode_operand_map(&map_b, 2, weights, d.n, d.k, pitch, false, BN, 1, 0)) return cudaErrorNotSupported;

  HalfConvParams p = {};
  p.status = tc_status_device();
  p.image = static_cast<const __half*>(d.a) + d.a_off;
  p.result = static_cast<__half*>(d.c) + d.c_off;
  p.image_stride = d.a_stride;
  p.result_stride = d.c_stride;
  p.m = static_cast<int>(d.m); p.n = static_cast<int>(d.n); p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>(tiles_m);
  p.tiles_n = static_cast<int>(tiles_n);
  p.k_blocks = static_cast<int>(k_blocks);
  p.batch = static_cast<int>(d.batch);
  p.conv = d.conv;

  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;
  int sms = device_sms;
  if (sm_budget() > 0 && sm_budget() < sms) sms = sm_budget();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(hconv_tc_kernel), static_cast<int>(smem));
  if (e != cudaSuccess) return e;
  *name = "tc_conv_f16_128x128x64_tmem_a";
  hconv_tc_kernel<<<grid, NUM_THREADS, static_cast<size_t>(smem), stream>>>(map_b, p);
  return cudaGetLastError();
}

}  // namespace b200
