// SGEMM as error-compensated 3xTF32 on CTA pairs: two SMs of a cluster share one 256 x 256 output tile
// (tcgen05.mma.cta_group::2 kind::tf32). The single-CTA kernel in gemm_tc_f32.cu is bound by shared-memory
// bandwidth (every K block is written by TMA, rewritten as TF32 big/small parts and read by twelve MMAs); with a
// pair each SM stages and splits only its own 128 rows of op(A) and its own 128 of the 256 columns of op(B),
// which takes a third off the bytes each shared memory moves per FLOP.
//
// Arithmetic, accuracy and the chunked accumulation are those of gemm_tc_f32.cu: x = hi + lo with hi = tf32(x),
// lo = tf32(x - hi); lo_a*hi_b + hi_a*lo_b + hi_a*hi_b accumulated by the tensor cores over 128 K into one of two
// TMEM partials, which the drain warps add into fp32 registers with round-to-nearest. Replaces the reference's
// indirect GEMM path (src/routines/level3/xgemm.cpp:101-222, src/kernels/level3/xgemm_part3.opencl:53-305) for large
// single-precision problems with TMA-compatible operands.
//
// Roles per CTA (640 threads): warp 0 TMA producer (own tiles, own barrier), warp 1 TMEM owner and - in the leader
// CTA - MMA issuer for the pair, warps 4-11 split (they arrive on the leader's "split done" barrier), warps 12-19
// drain + epilogue for this CTA's 128 rows (they arrive on the leader's "partial free" barrier). tcgen05.commit
// signals "stage free" and "partial full" in both CTAs. All waits are bounded; both CTAs meet at a cluster barrier
// before TMEM is released.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <cstring>

#include "../tc_host.h"
#include "launchers.h"
#include "../runtime_state.h"
#include "tc_common.cuh"

namespace b200 {

namespace {

using namespace tc;

constexpr int BM = 128;       // rows of op(A) per CTA; the pair covers 256
constexpr int BN_HALF = 128;  // columns of op(B) staged per CTA
constexpr int BN = 256;       // accumulator columns per CTA
constexpr int BK = 32;        // 32 floats = one 128-byte swizzle row
constexpr int UMMA_K = 8;
constexpr int NUM_THREADS = 640;
constexpr int LAUNCH_REGS = 96;
constexpr int PRODUCER_REGS = 40, SPLIT_REGS = 56, DRAIN_REGS = 160;
static_assert(128 * PRODUCER_REGS + 256 * SPLIT_REGS + 256 * DRAIN_REGS <= NUM_THREADS * LAUNCH_REGS,
              "register budgets exceed the CTA's pool");
constexpr int CHUNK_KB = 4;  // 128 K per partial: error 2^-24.3 * sum|a||b| at K = 8192 (64 K: 2^-25), 6 % faster at 4096^3
constexpr int TMEM_COLS = 512;
constexpr int A_BYTES = BM * BK * 4;
constexpr int B_BYTES = BN_HALF * BK * 4;
constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);  // main (raw -> hi in place) and lo copies
constexpr int STAGES = 3;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

struct PairParams {
  unsigned int* status;  // where an expired bounded wait is reported (mapped host memory), or null
  float* c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n, k_blocks;  // 256 x 256 pair tiles
  float alpha, beta;
  int raster_group;
  // batch: tiles of problem z follow those of problem z - 1; operands shared by all problems have *_batched == 0
  int batches, a_batched, b_batched;
  long long c_stride;
  const float* alphas;  // per-problem scalars (offset-table calls), or null
  const float* betas;
  // Rank-k updates (square C, one problem): 1 keeps the elements with row <= column, 2 those with row >= column.
  // Only the tiles that touch the triangle exist: they are numbered row by row through the triangle, so every
  // pair of SMs gets the same number of them.
  int tri;
};

__device__ __forceinline__ void tile_coords(const PairParams& p, int tile, int& tm, int& tn) {
  if (p.tri != 0) {
    // tile = r (r + 1) / 2 + c with c <= r: (r, c) is (tm, tn) in the lower triangle, (tn, tm) in the upper one
    int r = static_cast<int>((sqrtf(8.f * static_cast<float>(tile) + 1.f) - 1.f) * 0.5f);
    while (r * (r + 1) / 2 > tile) --r;
    while ((r + 1) * (r + 2) / 2 <= tile) ++r;
    const int c = tile - r * (r + 1) / 2;
    tm = p.tri == 2 ? r : c;
    tn = p.tri == 2 ? c : r;
    return;
  }
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
sgemm_3xtf32_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base_ptr + STAGES * STAGE_BYTES);
  const uint32_t bar_base = smem_u32(bars);
  // [0,S) raw data landed (own CTA), [S,2S) split done (leader's is used), [2S,3S) stage free (each CTA its own),
  // then 2 partial-full (each CTA its own), 2 partial-free (leader's is used)
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto split_full = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto stage_free = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto part_full = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
  auto part_free = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int tiles_per_problem = p.tri != 0 ? p.tiles_m * (p.tiles_m + 1) / 2 : p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * p.batches;
  const int pair_index = blockIdx.x >> 1;
  const int pair_count = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(split_full(s), 8);   // the four warps of one split group in each of the two CTAs
      mbar_init(stage_free(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(part_full(a), 1);
      mbar_init(part_free(a), 16);   // eight drain warps in each of the two CTAs
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // stage layout: A main | B main | A lo | B lo
  auto a_main = [&](int s) { return tiles_base + s * STAGE_BYTES; };
  auto b_main = [&](int s) { return a_main(s) + A_BYTES; };
  auto a_lo = [&](int s) { return b_main(s) + B_BYTES; };
  auto b_lo = [&](int s) { return a_lo(s) + A_BYTES; };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
    if (warp == 0) {
      // ---- TMA producer: this CTA's A rows and its half of the B columns, counted on this CTA's barrier ----
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        int issued = 0;
        bool ok = true;
        for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count) {
          int tm, tn;
          const int z = tile / tiles_per_problem;
          tile_coords(p, tile - z * tiles_per_problem, tm, tn);
          const int a_row0 = tm * 2 * BM + static_cast<int>(rank) * BM;
          const int b_row0 = tn * BN + static_cast<int>(rank) * BN_HALF;
          const int az = p.a_batched ? z : 0, bz = p.b_batched ? z : 0;
          for (int kb = 0; kb < p.k_blocks; ++kb) {
            if (!mbar_wait(stage_free(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
            mbar_arrive_expect_tx(raw_full(stage), A_BYTES + B_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 32; ++j)
                tma_load_3d(a_main(stage) + j * 4096, &map_a, raw_full(stage), a_row0 + j * 32, kb * BK, az);
            } else {
              tma_load_3d(a_main(stage), &map_a, raw_full(stage), kb * BK, a_row0, az);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN_HALF / 32; ++j)
                tma_load_3d(b_main(stage) + j * 4096, &map_b, raw_full(stage), b_row0 + j * 32, kb * BK, bz);
            } else {
              tma_load_3d(b_main(stage), &map_b, raw_full(stage), kb * BK, b_row0, bz);
            }
            ++issued;
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
        if (!ok) {
          const int pending = issued < STAGES ? issued : STAGES;
          for (int i = 0; i < pending; ++i) {
            const long long start = clock64();
            int s = stage - 1 - i;
            if (s < 0) s += STAGES;
            const uint32_t par = (s < stage) ? phase : (phase ^ 1u);
            while (!mbar_try_wait(raw_full(s), par) && clock64() - start < kWaitCycles / 8) {}
          }
        }
      }
    } else if (warp == 1) {
      // ---- MMA issuer: leader CTA only, for both SMs ----
      if (leader && lane == 0) {
        constexpr uint32_t idesc = make_idesc(2 * BM, BN, 2, A_MN ? 1 : 0, B_MN ? 1 : 0);
        int stage = 0;
        uint32_t phase = 0;
        int chunk_index = 0;
        bool ok = true;
        for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count) {
          for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += CHUNK_KB, ++chunk_index) {
            const int part = chunk_index & 1;
            const uint32_t part_phase = (chunk_index >> 1) & 1u;
            if (!mbar_wait_cluster(part_free(part), part_phase ^ 1u, abort_flag, 2u, p.status)) {
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(part * (TMEM_COLS / 2));
            const int kb_end = min(kb0 + CHUNK_KB, p.k_blocks);
            for (int kb = kb0; kb < kb_end; ++kb) {
              if (!mbar_wait_cluster(split_full(stage), phase, abort_flag, 3u, p.status)) {
                ok = false;
                break;
              }
              tcgen05_fence_after();
              const uint32_t a_lbo = A_MN ? 4096u : 16u, b_lbo = B_MN ? 4096u : 16u;
              const uint32_t a_sbo = A_MN ? 512u : 1024u, b_sbo = B_MN ? 512u : 1024u;
              const uint32_t a_type = A_MN ? kLayoutSw128Base32 : kLayoutSw128;
              const uint32_t b_type = B_MN ? kLayoutSw128Base32 : kLayoutSw128;
              const uint32_t a_step = A_MN ? 1024u : 32u, b_step = B_MN ? 1024u : 32u;
#pragma unroll
              for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                const uint64_t a_hi = smem_desc(a_main(stage) + ks * a_step, a_lbo, a_sbo, a_type);
                const uint64_t a_sm = smem_desc(a_lo(stage) + ks * a_step, a_lbo, a_sbo, a_type);
                const uint64_t b_hi = smem_desc(b_main(stage) + ks * b_step, b_lbo, b_sbo, b_type);
                const uint64_t b_sm = smem_desc(b_lo(stage) + ks * b_step, b_lbo, b_sbo, b_type);
                umma_tf32_pair(d_tmem, a_sm, b_hi, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);  // small terms first
                umma_tf32_pair(d_tmem, a_hi, b_sm, idesc, 1u);
                umma_tf32_pair(d_tmem, a_hi, b_hi, idesc, 1u);
              }
              umma_commit_pair(stage_free(stage));
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (ok) umma_commit_pair(part_full(part));
          }
        }
      }
    }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DRAIN_REGS));
    // ---- drain + epilogue: warp w reads TMEM lanes [32*(w%4), +32) and columns [128*h, +128) of its own CTA ----
    const int quad = warp & 3;
    const int half = (warp - 12) >> 2;
    int chunk_index = 0;
    bool ok = true;
    const uint32_t lead_free0 = map_to_cta(part_free(0), 0), lead_free1 = map_to_cta(part_free(1), 0);
    for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count) {
      int tm, tn;
      const int z = tile / tiles_per_problem;
      tile_coords(p, tile - z * tiles_per_problem, tm, tn);
      const float alpha = p.alphas ? p.alphas[z] : p.alpha;
      const float beta = p.betas ? p.betas[z] : p.beta;
      const bool use_beta = beta != 0.f;
      float acc[BN / 2];
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) acc[j] = 0.f;
      for (int kb0 = 0; kb0 < p.k_blocks; kb0 += CHUNK_KB, ++chunk_index) {
        const int part = chunk_index & 1;
        const uint32_t part_phase = (chunk_index >> 1) & 1u;
        ok = mbar_wait(part_full(part), part_phase, abort_flag, 4u, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               static_cast<uint32_t>(part * (TMEM_COLS / 2) + half * (BN / 2));
#pragma unroll
        for (int cb = 0; cb < BN / 64; ++cb) {
          uint32_t r[32];
          tmem_ld_32cols(t_row + cb * 32, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[cb * 32 + j] += __uint_as_float(r[j]);  // round-to-nearest adds
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(part ? lead_free1 : lead_free0);
      }
      if (!ok) break;
      const int row = tm * 2 * BM + static_cast<int>(rank) * BM + quad * 32 + lane;
      const int col0 = tn * BN + half * (BN / 2);
      if (row < p.m) {
        float* cptr = p.c + z * p.c_stride + static_cast<long long>(col0) * p.ldc + row;
        // Eight old values are fetched before the first store of a group: loads and stores through one pointer
        // would otherwise be serialised, one memory latency per element.
#pragma unroll
        for (int j0 = 0; j0 < BN / 2; j0 += 8) {
          float old[8];
          if (use_beta) {
#pragma unroll
            for (int jj = 0; jj < 8; ++jj)
              old[jj] = (col0 + j0 + jj < p.n) ? cptr[static_cast<long long>(j0 + jj) * p.ldc] : 0.f;
          }
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const int col = col0 + j0 + jj;
            if (col < p.n && (p.tri == 0 || (p.tri == 1 ? row <= col : row >= col))) {
              float v = __fmul_rn(alpha, acc[j0 + jj]);
              if (use_beta) v = fmaf(beta, old[jj], v);
              cptr[static_cast<long long>(j0 + jj) * p.ldc] = v;
            }
          }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SPLIT_REGS));
    // ---- split: warps 4..11 turn this CTA's raw fp32 tiles into TF32 big parts (in place) and small parts ----
    // Two groups of four warps take alternate K blocks, so the wait / fence / arrive latency of one stage overlaps
    // the conversion work of the next.
    const int t = threadIdx.x - 4 * 32;
    const int group = t >> 7, gt = t & 127;
    bool ok = true;
    constexpr int CHUNKS = (A_BYTES + B_BYTES) / 16;
    int kbg = 0;  // running K-block count of this CTA
    for (int tile = pair_index; tile < num_tiles && ok; tile += pair_count) {
      for (int kb = 0; kb < p.k_blocks; ++kb, ++kbg) {
        if ((kbg & 1) != group) continue;
        const int stage = kbg % STAGES;
        const uint32_t phase = static_cast<uint32_t>(kbg / STAGES) & 1u;
        ok = mbar_wait(raw_full(stage), phase, abort_flag, 5u, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        float4* const main_ptr = reinterpret_cast<float4*>(base_ptr + stage * STAGE_BYTES);
        float4* const lo_ptr = reinterpret_cast<float4*>(base_ptr + stage * STAGE_BYTES + A_BYTES + B_BYTES);
#pragma unroll 4
        for (int c = gt; c < CHUNKS; c += 128) {
          const float4 x = main_ptr[c];
          float4 hi, lo;
          hi.x = to_tf32_big(x.x); hi.y = to_tf32_big(x.y); hi.z = to_tf32_big(x.z); hi.w = to_tf32_big(x.w);
          lo.x = to_tf32(x.x - hi.x); lo.y = to_tf32(x.y - hi.y); lo.z = to_tf32(x.z - hi.z); lo.w = to_tf32(x.w - hi.w);
          main_ptr[c] = hi;
          lo_ptr[c] = lo;
        }
        fence_proxy_async();  // the tensor cores of both SMs read these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(split_full(stage), 0));
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody releases TMEM or exits while the peer may still signal or read
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN>
int resident_pairs() {
  auto kernel = sgemm_3xtf32_pair_kernel<A_MN, B_MN>;
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
cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const PairParams& p, long long tiles,
                           cudaStream_t stream) {
  auto kernel = sgemm_3xtf32_pair_kernel<A_MN, B_MN>;
  // The register re-balancing between warpgroups only works while the registers given to each thread at launch
  // cover the budgets asked for; otherwise leave the problem to the single-CTA kernels.
  int regs = 0;
  if (kernel_ready(reinterpret_cast<const void*>(kernel), SMEM_BYTES, &regs) != cudaSuccess) return cudaErrorNotSupported;
  if (regs < LAUNCH_REGS) return cudaErrorNotSupported;
  static std::atomic<int> pairs_of_device[kMaxDevices];
  int pairs = per_device(pairs_of_device, &resident_pairs<A_MN, B_MN>);
  if (pairs <= 0) return cudaErrorNotSupported;
  if (sm_budget() > 0 && sm_budget() / 2 < pairs) pairs = sm_budget() / 2;
  if (pairs <= 0) return cudaErrorNotSupported;
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  kernel<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_tc_f32_pair(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 32 || d.is_conv || d.force_small || d.conj_a || d.conj_b) return cudaErrorNotSupported;
  const BatchWalk walk = batch_walk(d);
  if (!walk.ok) return cudaErrorNotSupported;
  if (d.tri != 0 && (d.m != d.n || walk.batches != 1)) return cudaErrorNotSupported;
  // B200BLAS_SGEMM=ffma forces the CUDA-core kernel, =single the one-CTA-per-tile tensor-core kernels
  static const bool disabled = [] {
    const char* v = std::getenv("B200BLAS_SGEMM");
    return v != nullptr && (std::strcmp(v, "ffma") == 0 || std::strcmp(v, "single") == 0 || std::strcmp(v, "single128") == 0);
  }();
  if (disabled) return cudaErrorNotSupported;
  if (d.m < 512 || d.n < 256 || d.k < 128) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;
  const float* a = static_cast<const float*>(d.a) + d.a_off;
  const float* b = static_cast<const float*>(d.b) + d.b_off;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return cudaErrorNotSupported;
  if ((d.lda % 4) || (d.ldb % 4)) return cudaErrorNotSupported;
  if ((walk.a_stride % 4) || (walk.b_stride % 4)) return cudaErrorNotSupported;

  PairParams p;
  p.status = tc_status_device();
  p.batches = walk.batches;
  p.a_batched = walk.a_batches > 1;
  p.b_batched = walk.b_batches > 1;
  p.c_stride = walk.c_stride;
  p.alphas = static_cast<const float*>(d.alphas);
  p.betas = static_cast<const float*>(d.betas);
  p.c = static_cast<float*>(d.c) + d.c_off;
  p.ldc = d.ldc;
  p.m = static_cast<int>(d.m); p.n = static_cast<int>(d.n); p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>((d.m + 2 * BM - 1) / (2 * BM));
  p.tiles_n = static_cast<int>((d.n + BN - 1) / BN);
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  p.raster_group = 8;
  p.tri = d.tri;
  const long long tiles = d.tri != 0 ? static_cast<long long>(p.tiles_m) * (p.tiles_m + 1) / 2
                                     : static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  // Enough 256 x 256 tiles to give every pair of SMs two: below that the 128-wide single-CTA tiles fill the
  // machine better. (A rank-k update has no single-CTA tensor-core kernel to fall back to: one tile per pair is enough.)
  if (tiles < (d.tri != 0 ? sm_count() / 2 : sm_count()) || tiles > 0x7FFFFFFF) return cudaErrorNotSupported;

  CUtensorMap map_a, map_b;
  if (!encode_operand_map(&map_a, 4, a, d.m, d.k, d.lda, !d.a_kcontig, BM, walk.a_batches, walk.a_stride))
    return cudaErrorNotSupported;
  if (!encode_operand_map(&map_b, 4, b, d.n, d.k, d.ldb, !d.b_kcontig, BN_HALF, walk.b_batches, walk.b_stride))
    return cudaErrorNotSupported;

  *name = "tc_f32_3xtf32_pair_256x256x32";
  const bool a_mn = !d.a_kcontig, b_mn = !d.b_kcontig;
  if (a_mn) {
    return b_mn ? launch_variant<true, true>(map_a, map_b, p, tiles, stream)
                : launch_variant<true, false>(map_a, map_b, p, tiles, stream);
  }
  return b_mn ? launch_variant<false, true>(map_a, map_b, p, tiles, stream)
              : launch_variant<false, false>(map_a, map_b, p, tiles, stream);
}

}  // namespace b200
