// HGEMM on the 5th-generation tensor cores: TMA -> shared-memory ring -> tcgen05.mma (kind::f16, fp32 accumulators
// in TMEM) -> tcgen05.ld epilogue. Persistent, warp-specialised, one CTA per SM.
//
// This kernel replaces, for half precision, the reference's "indirect" GEMM path: the Xgemm kernel plus its
// copy/pad/transpose pre- and post-kernels and the temporary buffers they need
// (src/routines/level3/xgemm.cpp:101-222, src/kernels/level3/xgemm_part3.opencl:53-305, copy_pad.opencl,
// transpose_pad.opencl). Edge tiles are zero-filled by the TMA unit and masked in the epilogue, so nothing is
// padded or transposed in memory. The reference accumulates half GEMMs in half; here products are exact and
// sums are fp32, rounded to half once (alpha*acc + beta*c is evaluated in fp32).
//
// Operand requirements (checked on the host, otherwise the CUDA-core kernel runs): 16-byte aligned base addresses
// and leading dimensions that are multiples of 8 elements. Both operand orientations are consumed where they lie
// (K-major tiles for K-contiguous operands, MN-major column blocks otherwise); nothing is transposed in memory.
//
// Roles per CTA (192 threads): warp 0 lane 0 issues TMA loads; warp 1 owns TMEM and lane 0 issues the MMAs;
// warps 2-5 drain accumulators (each warp reads the 32 TMEM lanes its rank modulo 4 may access).
// Every wait is bounded: on expiry the CTA records a code in the status block, all roles leave their loops, copies
// already in flight are waited for (bounded again), TMEM is released and the kernel returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>


#include "../tc_host.h"
#include "launchers.h"
#include "../runtime_state.h"
#include "hgemm_epilogue.cuh"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int BM = 128;      // MMA M: rows of op(A) per tile (TMEM lanes)
constexpr int BN = 256;      // MMA N: columns of op(B) per tile (TMEM columns per accumulator)
constexpr int BK = 64;       // K per stage: 64 halves = one 128-byte swizzle row
constexpr int UMMA_K = 16;   // K per tcgen05.mma for 16-bit inputs
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;  // two accumulators of BN fp32 columns
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + kStageBuffers * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

// [0] first timeout code seen (0 = none), [1] block that saw it, [2] role-specific detail.
struct TcParams {
  unsigned int* status;  // where an expired bounded wait is reported (mapped host memory), or null
  __half* c;
  long long ldc;
  int m, n, k;          // normalised extents: C is m x n with m contiguous
  int tiles_m, tiles_n;
  int k_blocks;
  float alpha, beta;
  int raster_group;     // m-tiles per rasterisation group
  // batch: tiles of problem z follow those of problem z - 1; operands shared by all problems have *_batched == 0
  int batches, a_batched, b_batched;
  long long c_stride;
  const float* alphas;  // per-problem scalars (offset-table calls), or null
  const float* betas;
  int c_by_tma;         // C goes out through the staging buffers and TMA stores
};

// Tiles are walked in groups of `raster_group` m-tiles by all n-tiles, m fastest inside a group, so the CTAs
// running at the same time share a small set of operand rows in L2.
__device__ __forceinline__ void tile_coords(const TcParams& p, int tile, int& tm, int& tn) {
  const int per_group = p.raster_group * p.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * p.raster_group;
  const int rows = min(p.raster_group, p.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

// A_MN / B_MN: the operand is M/N-contiguous and is loaded as 64-element-wide MN-major column blocks (one 128-byte
// row per k) instead of one K-major tile (128-byte rows along K).
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
hgemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint8_t* const staging = base_ptr + STAGES * STAGE_BYTES;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(staging + kStageBuffers * kStageBytes);
  // barrier slots: [0,S) full, [S,2S) empty, [2S,2S+2) accumulator full, [2S+2,2S+4) accumulator empty
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * p.batches;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    for (int b = 0; b < kStageBuffers; ++b) mbar_init(bar_base + 192u + 8u * b, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;  // stages armed so far (bounded by STAGES for the teardown wait)
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        const int z = tile / tiles_per_problem;
        tile_coords(p, tile - z * tiles_per_problem, tm, tn);
        const int az = p.a_batched ? z : 0, bz = p.b_batched ? z : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
          const uint32_t a_dst = tiles_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
          if (A_MN) {  // column blocks of 64 rows x 64 k = 8 KB each
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(a_dst + j * 8192, &map_a, full_bar(stage), tm * BM + j * 64, kb * BK, az);
          } else {
            tma_load_3d(a_dst, &map_a, full_bar(stage), kb * BK, tm * BM, az);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * 8192, &map_b, full_bar(stage), tn * BN + j * 64, kb * BK, bz);
          } else {
            tma_load_3d(b_dst, &map_b, full_bar(stage), kb * BK, tn * BN, bz);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Abort path: the copies already issued still land in shared memory; give each armed stage a bounded
        // chance to complete before the CTA may exit.
        const int pending = issued < STAGES ? issued : STAGES;
        for (int i = 0; i < pending; ++i) {
          const long long start = clock64();
          int s = stage - 1 - i;
          if (s < 0) s += STAGES;
          const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
          while (!mbar_try_wait(full_bar(s), par) && clock64() - start < kWaitCycles / 8) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 0, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_flag, 2u, p.status)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, 3u, p.status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_src = tiles_base + stage * STAGE_BYTES;
          const uint32_t b_src = a_src + A_BYTES;
          // K-major: 128-byte rows along K, advance 16 halves = 32 B per MMA. MN-major: one 128-byte row of 64
          // elements per k, swizzle atoms of eight k (1024 B, the stride offset), column blocks 8192 B apart (the
          // leading offset), advance 16 k = 2048 B per MMA.
          const uint64_t da = smem_desc(a_src, A_MN ? 8192 : 16, 1024, kLayoutSw128);
          const uint64_t db = smem_desc(b_src, B_MN ? 8192 : 16, 1024, kLayoutSw128);
          constexpr uint32_t a_step = A_MN ? (2048u >> 4) : 2u, b_step = B_MN ? (2048u >> 4) : 2u;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            umma_f16(d_tmem, da + a_step * ks, db + b_step * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the stage once the MMAs above have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(acc_full_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ---- epilogue: warps 2..5 ----
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
    const int row_in_cta = quad * 32 + lane;
    const bool elected = threadIdx.x == 64;  // first epilogue thread: issues and tracks the TMA stores
    int local = 0;
    int stores = 0;
    bool ok = true;
    HalfEpilogue e;
    e.ldc = p.ldc; e.m = p.m; e.n = p.n;
    e.use_tma = p.c_by_tma != 0;
    e.map_c = &map_c;
    e.staging = staging;
    e.load_bars = bar_base + 192u;
    e.hint_store = false;
    e.store_policy = e.hint_store ? l2_policy(1) : 0;
    uint32_t phases = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int tm, tn;
      const int z = tile / tiles_per_problem;
      tile_coords(p, tile - z * tiles_per_problem, tm, tn);
      e.alpha = p.alphas ? p.alphas[z] : p.alpha;
      e.beta = p.betas ? p.betas[z] : p.beta;
      e.c = p.c + z * p.c_stride;
      e.z = z;
      const int cta_row0 = tm * BM;
      const int col0 = tn * BN;
      // old values only matter where something is stored: CTAs wholly below C skip them
      const bool use_beta = e.beta != 0.f && cta_row0 < p.m;
      if (elected && e.use_tma && use_beta) prefetch_first_blocks(e, stores, cta_row0, col0);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1u;
      ok = mbar_wait(acc_full_bar(acc), acc_phase, abort_flag, 4u, p.status);
      ok = epilogue_all(ok);  // all four warps go on, or none
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; ++cb) {
        if (col0 + cb * 32 >= p.n) break;  // uniform over the CTA
        uint32_t r[32];
        tmem_ld_32cols(t_row + cb * 32, r);
        const int ahead = col0 + (cb + 2) * 32;
        if (!write_block(e, r, cta_row0 + row_in_cta, row_in_cta, cta_row0, col0 + cb * 32,
                         (cb + 2 < BN / 32 && ahead < p.n) ? ahead : -1, use_beta, stores, phases, elected, p.status)) {
          ok = false;
          break;
        }
      }
      if (!ok) break;
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
    }
    if (elected) bulk_wait_all();  // shared memory stays valid until the last store has read it
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const TcParams& p,
                           int grid, cudaStream_t stream) {
  auto kernel = hgemm_tc_kernel<A_MN, B_MN>;
  // per-context opt-in to more than 48 KB of dynamic shared memory (remembered per context)
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), SMEM_BYTES);
  if (e != cudaSuccess) return e;
  kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, mc, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_tc_f16(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 16 || d.is_conv || d.force_small || d.tri) return cudaErrorNotSupported;
  const BatchWalk walk = batch_walk(d);
  if (!walk.ok) return cudaErrorNotSupported;
  if (d.m < 128 || d.n < 64 || d.k < 64) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;
  const __half* a = static_cast<const __half*>(d.a) + d.a_off;
  const __half* b = static_cast<const __half*>(d.b) + d.b_off;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return cudaErrorNotSupported;
  if ((d.lda % 8) || (d.ldb % 8)) return cudaErrorNotSupported;

  CUtensorMap map_a, map_b;
  if (!encode_operand_map(&map_a, 2, a, d.m, d.k, d.lda, !d.a_kcontig, BM, walk.a_batches, walk.a_stride))
    return cudaErrorNotSupported;
  if (!encode_operand_map(&map_b, 2, b, d.n, d.k, d.ldb, !d.b_kcontig, BN, walk.b_batches, walk.b_stride))
    return cudaErrorNotSupported;

  TcParams p;
  p.status = tc_status_device();
  p.batches = walk.batches;
  p.a_batched = walk.a_batches > 1;
  p.b_batched = walk.b_batches > 1;
  p.c_stride = walk.c_stride;
  p.alphas = static_cast<const float*>(d.alphas);
  p.betas = static_cast<const float*>(d.betas);
  p.c = static_cast<__half*>(d.c) + d.c_off;
  p.ldc = d.ldc;
  p.m = static_cast<int>(d.m);
  p.n = static_cast<int>(d.n);
  p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>((d.m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((d.n + BN - 1) / BN);
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  p.raster_group = 16;

  // SM count is cached per device; the opt-in to more than 48 KB of dynamic shared memory is per context, and
  // contexts come and go, so it is simply repeated before every launch (a host-side attribute write).
  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;
    const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  if (tiles > 0x7FFFFFFF) return cudaErrorNotSupported;
  int sms = device_sms;
  if (sm_budget() > 0 && sm_budget() < sms) sms = sm_budget();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  CUtensorMap map_c;
  p.c_by_tma = encode_half_c_map(&map_c, p.c, d.m, d.n, d.ldc, walk.batches, walk.c_stride) ? 1 : 0;
  if (!p.c_by_tma) std::memset(&map_c, 0, sizeof(map_c));
  *name = "tc_f16_128x256x64";
  const bool a_mn = !d.a_kcontig, b_mn = !d.b_kcontig;
  if (a_mn) {
    return b_mn ? launch_variant<true, true>(map_a, map_b, map_c, p, grid, stream)
                : launch_variant<true, false>(map_a, map_b, map_c, p, grid, stream);
  }
  return b_mn ? launch_variant<false, true>(map_a, map_b, map_c, p, grid, stream)
              : launch_variant<false, false>(map_a, map_b, map_c, p, grid, stream);
}

}  // namespace b200
