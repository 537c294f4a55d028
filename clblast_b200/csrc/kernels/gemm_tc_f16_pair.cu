// HGEMM on CTA pairs: two SMs of a thread-block cluster work on one 256 x 256 output tile with
// tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of op(A) and its own 128 of the 256 columns of op(B);
// the tensor cores of both SMs read the two B halves from both shared memories, so every operand byte is loaded
// from L2 once per pair instead of once per SM, and each SM's shared memory takes 32 KB per K block instead of 48.
//
// Same contract as the single-CTA kernel in gemm_tc_f16.cu (which stays the path for problems with fewer than 256
// rows): replaces the reference's indirect GEMM path for half precision (src/routines/level3/xgemm.cpp:101-222,
// src/kernels/level3/xgemm_part3.opencl:53-305), fp32 accumulation, alpha*acc + beta*c evaluated in fp32 and
// rounded to half once, edge tiles zero-filled by TMA and masked in the epilogue.
//
// Roles per CTA (192 threads): warp 0 lane 0 issues this CTA's TMA loads, which signal the LEADER CTA's "full"
// barrier; warp 1 allocates TMEM (pair-wide allocation, executed in both CTAs) and, in the leader CTA only, lane 0
// issues the MMAs for the pair; warps 2-5 of both CTAs drain their CTA's 128 accumulator rows. tcgen05.commit
// signals the "stage free" and "accumulator full" barriers of both CTAs; the epilogue warps of both CTAs arrive on
// the leader's "accumulator free" barrier.
// Every wait is bounded (a code is left in the status word, all roles leave their loops); both CTAs meet at a
// cluster barrier before TMEM is released, so no CTA signals a peer that has already exited.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>

#include "../tc_host.h"
#include "launchers.h"
#include "../runtime_state.h"
#include "hgemm_epilogue.cuh"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int BM = 128;        // rows of op(A) per CTA (TMEM lanes); the pair covers 256
constexpr int BN_HALF = 128;   // columns of op(B) staged per CTA
constexpr int BN = 256;        // MMA N: accumulator columns in each CTA's TMEM
constexpr int BK = 64;         // 64 halves = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN_HALF * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;  // two accumulators of 256 fp32 columns
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + kStageBuffers * kStageBytes + 1024 + 256;

struct PairParams {
  unsigned int* status;  // where an expired bounded wait is reported (mapped host memory), or null
  __half* c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n;  // in 256 x 256 pair tiles
  int k_blocks;
  float alpha, beta;
  int raster_group;
  // batch: tiles of problem z follow those of problem z - 1; operands shared by all problems have *_batched == 0
  int batches, a_batched, b_batched;
  long long c_stride;
  const float* alphas;  // per-problem scalars (offset-table calls), or null
  const float* betas;
  int c_by_tma;         // C goes out through the staging buffers and TMA stores
  int hint_a, hint_b;   // L2 eviction priority of the operand loads (0 normal, 1 evict-first, 2 evict-last)
  int hint_c;           // result stores are marked evict-first
};

__device__ __forceinline__ void tile_coords(const PairParams& p, int tile, int& tm, int& tn) {
  const int per_group = p.raster_group * p.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * p.raster_group;
  const int rows = min(p.raster_group, p.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
hgemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_c, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint8_t* const staging = base_ptr + STAGES * STAGE_BYTES;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(staging + kStageBuffers * kStageBytes);
  const uint32_t bar_base = smem_u32(bars);
  // [0,S) full (used in the leader), [S,2S) empty (each CTA its own), then accumulator full x2 (each CTA its own),
  // accumulator empty x2 (used in the leader)
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * p.batches;
  const int pair_index = blockIdx.x >> 1;
  const int pair_count = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);  // four epilogue warps in each of the two CTAs
    }
    for (int b = 0; b < kStageBuffers; ++b) mbar_init(bar_base + 192u + 8u * b, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals across the pair
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer (both CTAs): own A rows, own half of the B columns ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_a = l2_policy(p.hint_a), pol_b = l2_policy(p.hint_b);
      for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count) {
        int tm, tn;
        const int z = tile / tiles_per_problem;
        tile_coords(p, tile - z * tiles_per_problem, tm, tn);
        const int a_row0 = tm * 2 * BM + static_cast<int>(rank) * BM;
        const int b_row0 = tn * BN + static_cast<int>(rank) * BN_HALF;
        const int az = p.a_batched ? z : 0, bz = p.b_batched ? z : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
          const uint32_t a_dst = tiles_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);  // the bytes of both CTAs
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d_pair_hint(a_dst + j * 8192, &map_a, lead_full, a_row0 + j * 64, kb * BK, az, pol_a);
          } else {
            tma_load_3d_pair_hint(a_dst, &map_a, lead_full, kb * BK, a_row0, az, pol_a);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN_HALF / 64; ++j)
              tma_load_3d_pair_hint(b_dst + j * 8192, &map_b, lead_full, b_row0 + j * 64, kb * BK, bz, pol_b);
          } else {
            tma_load_3d_pair_hint(b_dst, &map_b, lead_full, kb * BK, b_row0, bz, pol_b);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Abort path: copies already issued still land in this CTA's shared memory; their completion is counted in
        // the leader, so wait a bounded time (far longer than any copy takes) before the CTA may leave.
        const long long start = clock64();
        while (clock64() - start < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: leader CTA only, for both SMs ----
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc(2 * BM, BN, 0, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count, ++local) {
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
          // K-major: 128-byte rows along K (stride offset 1024 = eight rows), 32 B per MMA step. MN-major: one
          // 128-byte row of 64 elements per k, column blocks 8192 B apart, 2048 B per MMA step.
          const uint64_t da = A_MN ? smem_desc(a_src, 8192, 1024, kLayoutSw128) : smem_desc(a_src, 16, 1024, kLayoutSw128);
          const uint64_t db = B_MN ? smem_desc(b_src, 8192, 1024, kLayoutSw128) : smem_desc(b_src, 16, 1024, kLayoutSw128);
          constexpr uint32_t a_step = A_MN ? (2048u >> 4) : 2u, b_step = B_MN ? (2048u >> 4) : 2u;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            umma_f16_pair(d_tmem, da + a_step * ks, db + b_step * ks, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));  // frees this stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(acc_full_bar(acc));  // both CTAs' epilogues may read this accumulator
      }
    }
  } else {
    // ---- epilogue: warps 2..5 of both CTAs, 128 rows x 256 columns each ----
    const int quad = warp & 3;
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
    e.hint_store = (p.hint_c != 0);
    e.store_policy = e.hint_store ? l2_policy(1) : 0;
    uint32_t phases = 0;
    for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count, ++local) {
      int tm, tn;
      const int z = tile / tiles_per_problem;
      tile_coords(p, tile - z * tiles_per_problem, tm, tn);
      e.alpha = p.alphas ? p.alphas[z] : p.alpha;
      e.beta = p.betas ? p.betas[z] : p.beta;
      e.c = p.c + z * p.c_stride;
      e.z = z;
      const int cta_row0 = tm * 2 * BM + static_cast<int>(rank) * BM;
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
      if (lane == 0) mbar_arrive_remote(map_to_cta(acc_empty_bar(acc), 0));
    }
    if (elected) bulk_wait_all();  // shared memory stays valid until the last store has read it
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody releases TMEM or exits while the peer may still signal or read
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Number of CTA pairs the device can hold at once (one CTA per SM; pairs must sit in one GPC).
template <bool A_MN, bool B_MN>
int resident_pairs() {
  auto kernel = hgemm_tc_pair_kernel<A_MN, B_MN>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

template <bool A_MN, bool B_MN>
cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const PairParams& p,
                           long long tiles, cudaStream_t stream) {
  auto kernel = hgemm_tc_pair_kernel<A_MN, B_MN>;
  static std::atomic<int> pairs_of_device[kMaxDevices];
  int pairs = per_device(pairs_of_device, &resident_pairs<A_MN, B_MN>);
  if (pairs <= 0) return cudaErrorNotSupported;
  if (sm_budget() > 0 && sm_budget() / 2 < pairs) pairs = sm_budget() / 2;
  if (pairs <= 0) return cudaErrorNotSupported;
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), SMEM_BYTES);
  if (e != cudaSuccess) return e;
  kernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, mc, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_tc_f16_pair(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 16 || d.is_conv || d.force_small || d.tri) return cudaErrorNotSupported;
  const BatchWalk walk = batch_walk(d);
  if (!walk.ok) return cudaErrorNotSupported;
  // B200BLAS_HGEMM=single keeps the one-CTA-per-tile kernel
  static const bool forced_single = [] {
    const char* v = std::getenv("B200BLAS_HGEMM");
    return v != nullptr && std::strcmp(v, "single") == 0;
  }();
  if (forced_single) return cudaErrorNotSupported;
  if (d.m < 256 || d.n < 128 || d.k < 64) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;
  const __half* a = static_cast<const __half*>(d.a) + d.a_off;
  const __half* b = static_cast<const __half*>(d.b) + d.b_off;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return cudaErrorNotSupported;
  if ((d.lda % 8) || (d.ldb % 8)) return cudaErrorNotSupported;

  PairParams p;
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
  p.tiles_m = static_cast<int>((d.m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = static_cast<int>((d.n + BN - 1) / BN);
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  // Tile order and L2 priorities; the environment variables exist for tuning runs.
  static const int raster_env = [] { const char* v = std::getenv("B200BLAS_HGEMM_RASTER"); return v ? std::atoi(v) : 0; }();
  static const int hint_env = [] { const char* v = std::getenv("B200BLAS_HGEMM_L2HINT"); return v ? std::atoi(v) : -1; }();
  p.raster_group = raster_env > 0 ? raster_env : 8;
  // Default: both operands evict-last (panels are re-read by the tiles that share them; measured +2 to 3 % over
  // normal priority at 8192^3). The variable takes three digits: A, B, and 1 for evict-first result stores.
  const int hints = hint_env >= 0 ? hint_env : 220;
  p.hint_a = (hints / 100) % 10;
  p.hint_b = (hints / 10) % 10;
  p.hint_c = hints % 10;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  if (tiles > 0x7FFFFFFF) return cudaErrorNotSupported;
  // Half-empty pair tiles waste a whole SM: leave problems whose last row of pair tiles is at most half full, and
  // that have few tiles, to the single-CTA kernel.
  const long long single_tiles = ((d.m + BM - 1) / BM) * p.tiles_n * p.batches;
  if (single_tiles < 2 * tiles && tiles < sm_count()) return cudaErrorNotSupported;

  CUtensorMap map_a, map_b;
  if (!encode_operand_map(&map_a, 2, a, d.m, d.k, d.lda, !d.a_kcontig, BM, walk.a_batches, walk.a_stride))
    return cudaErrorNotSupported;
  if (!encode_operand_map(&map_b, 2, b, d.n, d.k, d.ldb, !d.b_kcontig, BN_HALF, walk.b_batches, walk.b_stride))
    return cudaErrorNotSupported;

  CUtensorMap map_c;
  p.c_by_tma = encode_half_c_map(&map_c, p.c, d.m, d.n, d.ldc, walk.batches, walk.c_stride) ? 1 : 0;
  if (!p.c_by_tma) std::memset(&map_c, 0, sizeof(map_c));

  *name = "tc_f16_pair_256x256x64";
  const bool a_mn = !d.a_kcontig, b_mn = !d.b_kcontig;
  if (a_mn) {
    return b_mn ? launch_variant<true, true>(map_a, map_b, map_c, p, tiles, stream)
                : launch_variant<true, false>(map_a, map_b, map_c, p, tiles, stream);
  }
  return b_mn ? launch_variant<false, true>(map_a, map_b, map_c, p, tiles, stream)
              : launch_variant<false, false>(map_a, map_b, map_c, p, tiles, stream);
}

}  // namespace b200
