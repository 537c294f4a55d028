// SGEMM on the tensor cores with fp32-level accuracy: error-compensated 3xTF32 (TMA -> split into TF32 "big" and
// "small" parts in shared memory -> three tcgen05.mma kind::tf32 per K step with fp32 accumulators in TMEM).
//
// Replaces, for large single-precision GEMMs with TMA-compatible operands, the reference's indirect path (Xgemm
// kernel plus copy/pad/transpose kernels and temporaries: src/routines/level3/xgemm.cpp:101-222,
// src/kernels/level3/xgemm_part3.opencl:53-305). Each fp32 operand x is split as x = hi + lo + e with
// hi = tf32(x), lo = tf32(x - hi), both exactly representable in TF32 and |e| <= 2^-22 |x|; the product is formed as
// lo_a*hi_b + hi_a*lo_b + hi_a*hi_b (the lo*lo term, <= 2^-22 relative, is dropped). The tensor cores add into
// their fp32 accumulators with truncation, which over thousands of accumulations costs several bits, so they only
// accumulate over a short chunk of K (CHUNK_KB blocks of 32) into one of two TMEM partial buffers; eight
// "drain" warps then add each finished partial into fp32 register accumulators with round-to-nearest while the
// tensor cores fill the other buffer. The result is not bit-identical to the k-ascending fused multiply-add chain
// of the CUDA-core kernel; its error against the fp64 product stays at the fp32 level (asserted in the tests).
//
// Both operand orientations are consumed where they lie: a K-contiguous operand is loaded as one K-major tile, an
// M/N-contiguous operand as 32-wide MN-major column blocks; the split is element-wise and in place, so no transpose
// ever happens. Non-finite inputs: an infinite operand yields a non-finite result in every output it touches, but
// it may be NaN where plain fp32 arithmetic gives +-inf (inf times a negative small part); the reference's own
// comparison rule treats the two alike (test/correctness/tester.cpp:569-577).
// Operands whose base is 16-byte aligned and whose leading dimension is a multiple of 4 elements travel by TMA;
// any other operand pair is gathered by the split warps with coalesced scalar loads (bounds-checked, so every
// offset and leading dimension is accepted) and written straight into the swizzled big/small tiles.
//
// Roles (640 threads, five warpgroups with re-balanced register budgets): warp 0 TMA producer, warp 1 MMA issuer
// and TMEM owner (warps 2-3 idle), warps 4-11 split, warps 12-19 drain + epilogue.
// All waits are bounded; on expiry a code is left in the status block and the CTA drains and exits.
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

constexpr int BM = 128;
constexpr int BK = 32;  // 32 floats = one 128-byte swizzle row
constexpr int UMMA_K = 8;
constexpr int NUM_THREADS = 640;
// Register re-balancing must stay inside the CTA's own allocation (threads x registers at launch), otherwise the
// increase waits forever: 128 producer threads x 40 + 256 split threads x 56 + 256 drain threads x 160.
constexpr int LAUNCH_REGS = 96;  // floor(65536 / 640) rounded down to the allocation granularity of 8
static_assert(128 * 40 + 256 * 56 + 256 * 160 <= NUM_THREADS * LAUNCH_REGS, "register budgets exceed the CTA's pool");
constexpr int CHUNK_KB = 4;  // K blocks accumulated inside the tensor cores before a partial is drained
constexpr int TMEM_COLS = 512;

struct Tc32Params {
  unsigned int* status;  // where an expired bounded wait is reported (mapped host memory), or null
  float* c;
  long long ldc;
  int m, n, k;
  int tiles_m, tiles_n, k_blocks;
  float alpha, beta;
  int raster_group;
  // GEMM batch: tiles of problem z follow those of problem z - 1; operands shared by all problems have *_batched == 0
  int batches, a_batched, b_batched;
  long long a_stride, b_stride, gemm_c_stride;
  const float* alphas;  // per-problem scalars (offset-table calls), or null
  const float* betas;
  // The kernel computes the transposed problem (operands swapped by the launcher): element (row, col) of its tile
  // goes to c[row * ldc + col], so each thread's results are contiguous in memory. c_vec4: 16-byte stores allowed.
  int c_rowmajor, c_vec4;
  // gathered operands (no TMA): element pointers and leading dimensions
  const float* a;
  const float* b;
  long long lda, ldb;
  // convolution only: op(A) is gathered from the image, one GEMM per image
  const float* image;
  long long image_stride, c_stride;
  int batch;
  ConvGeom conv;
  // Division-free gather (rows of at least eight output pixels, offsets that fit 32 bits): kg / (kernel_h * kernel_w)
  // and tap / kernel_w become multiply-high by these constants (0: the divisor is 1).
  int conv_fast;
  unsigned khw_magic, kw_magic;
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int MAIN_BYTES = A_BYTES + B_BYTES;  // one K block: raw fp32, turned into the big parts in place
  // The big-part ring is held from the TMA issue until the MMAs have read it, so its depth is what hides the load
  // latency; a small-part tile only lives from the split to the MMAs, so a shorter ring of its own is enough - but not
  // much shorter: split -> MMA -> commit -> next split is a serial chain per slot (measured with 128x64 tiles: load
  // ring 7 + 2 slots: 1024^3 35.6 us, 2048 x (64x128x96) 87 us; 6 + 3: 29.8 / 75.6 us; 4 + 4, the coupled ring this
  // replaces: 30.0 / 64.7 us).
  static constexpr int STAGES = (BN == 256) ? 2 : (BN == 64) ? 5 : 4;
  static constexpr int LO_STAGES = (BN == 256) ? 2 : (BN == 64) ? 4 : 3;
  static constexpr int SMEM_BYTES = (STAGES + LO_STAGES) * MAIN_BYTES + 1024 + 512;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
};

// Convolution tiles: m fastest, then n, then the image index.
__device__ __forceinline__ void conv_tile_coords(const Tc32Params& p, int tile, int& tm, int& tn, int& image) {
  tm = tile % p.tiles_m;
  const int rest = tile / p.tiles_m;
  tn = rest % p.tiles_n;
  image = rest / p.tiles_n;
}

__device__ __forceinline__ void tile_coords(const Tc32Params& p, int tile, int& tm, int& tn) {
  const int per_group = p.raster_group * p.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * p.raster_group;
  const int rows = min(p.raster_group, p.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

// A_MN / B_MN: the operand is M/N-contiguous (MN-major tiles) instead of K-contiguous (K-major tiles).
// MODE kConv: op(A) is the implicit im2col matrix of one image (rows = output pixels, always MN-major); the split
// warps gather it straight from the image into the swizzled big/small tiles, so only B (the weights) travels by TMA.
// MODE kGather: both operands are gathered by the split warps; the TMA warp only forwards "stage free".
constexpr int kTma = 0, kConv = 1, kGather = 2;
template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sgemm_3xtf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const Tc32Params p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  constexpr int LO_STAGES = C::LO_STAGES;
  constexpr bool CONV = MODE == kConv;
  constexpr bool GATHER = MODE == kGather;
  static_assert(!GATHER || BN == 128, "the gathered variant prefetches 16 + 16 values per thread");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint64_t* const bars = reinterpret_cast<uint64_t*>(base_ptr + (STAGES + LO_STAGES) * C::MAIN_BYTES);
  const uint32_t bar_base = smem_u32(bars);
  // [0,S) raw data landed, [S,2S) split done, [2S,3S) stage free, then 2 partial-full, 2 partial-free, L small-part
  // slot free
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto split_full = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto stage_free = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto part_full = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
  auto part_free = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
  auto lo_free = [&](int l) { return bar_base + 8u * (3 * STAGES + 4 + l); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4 + LO_STAGES);
  static_assert((3 * STAGES + 4 + LO_STAGES) * 8 + 8 <= 512, "barrier block");
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * (CONV ? p.batch : p.batches);
  // GEMM tiles: problem index, then the rasterised position inside the problem
  auto gemm_tile = [&](int tile, int& tm, int& tn, int& z) {
    z = tile / tiles_per_problem;
    tile_coords(p, tile - z * tiles_per_problem, tm, tn);
  };
  // register budgets (split, drain): the convolution variant prefetches its gather in registers and drains 64
  // columns per thread
  constexpr int SPLIT_REGS = (CONV || GATHER) ? 88 : 56;
  constexpr int DRAIN_REGS = (CONV || GATHER) ? 104 : 160;
  static_assert(128 * 40 + 256 * SPLIT_REGS + 256 * DRAIN_REGS <= NUM_THREADS * LAUNCH_REGS, "register budgets");

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(split_full(s), MODE == kTma ? 4 : 8);  // arrivals: one per warp of the group that splits the stage
      mbar_init(stage_free(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(part_full(a), 1);
      mbar_init(part_free(a), 8);
    }
    for (int l = 0; l < LO_STAGES; ++l) mbar_init(lo_free(l), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // layout: STAGES x (A main | B main), then LO_STAGES x (A lo | B lo); K block g of this CTA uses main stage
  // g % STAGES and small-part slot g % LO_STAGES
  auto a_main = [&](int s) { return tiles_base + s * C::MAIN_BYTES; };
  auto b_main = [&](int s) { return a_main(s) + C::A_BYTES; };
  auto a_lo = [&](int l) { return tiles_base + (STAGES + l) * C::MAIN_BYTES; };
  auto b_lo = [&](int l) { return a_lo(l) + C::A_BYTES; };
  uint8_t* const lo_ring = base_ptr + STAGES * C::MAIN_BYTES;

  // Register budgets are re-balanced per warpgroup: producers need few, drain warps hold 128 accumulators each.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int slot = 0;  // convolution: small-part slot the weights' small parts are loaded into
      uint32_t slot_phase = 0;
      int issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn, image_index = 0, z = 0;
        if (CONV) conv_tile_coords(p, tile, tm, tn, image_index); else gemm_tile(tile, tm, tn, z);
        const int az = p.a_batched ? z : 0, bz = p.b_batched ? z : 0;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(stage_free(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
          if (CONV && !mbar_wait(lo_free(slot), slot_phase ^ 1u, abort_flag, 8u, p.status)) { ok = false; break; }
          if (GATHER) {
            mbar_arrive(raw_full(stage));  // nothing to load: tell the split warps the stage is theirs
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          mbar_arrive_expect_tx(raw_full(stage), CONV ? 2 * C::B_BYTES : C::A_BYTES + C::B_BYTES);
          if (CONV) {
            // op(A) is gathered by the split warps; the weights were split once for all tiles (map_b: big parts,
            // map_a: small parts) and go straight to where the MMAs read them
            tma_load_3d(b_lo(slot), &map_a, raw_full(stage), kb * BK, tn * BN, 0);
            if (++slot == LO_STAGES) { slot = 0; slot_phase ^= 1u; }
          } else if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j)
              tma_load_3d(a_main(stage) + j * 4096, &map_a, raw_full(stage), tm * BM + j * 32, kb * BK, az);
          } else {
            tma_load_3d(a_main(stage), &map_a, raw_full(stage), kb * BK, tm * BM, az);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_3d(b_main(stage) + j * 4096, &map_b, raw_full(stage), tn * BN + j * 32, kb * BK, bz);
          } else {
            tma_load_3d(b_main(stage), &map_b, raw_full(stage), kb * BK, tn * BN, bz);
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
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 2, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int lo = 0;           // small-part slot of the current K block
      int chunk_index = 0;  // running count of partials produced by this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += CHUNK_KB, ++chunk_index) {
          const int part = chunk_index & 1;
          const uint32_t part_phase = (chunk_index >> 1) & 1u;
          if (!mbar_wait(part_free(part), part_phase ^ 1u, abort_flag, 2u, p.status)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(part * (TMEM_COLS / 2));
          const int kb_end = min(kb0 + CHUNK_KB, p.k_blocks);
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!mbar_wait(split_full(stage), phase, abort_flag, 3u, p.status)) { ok = false; break; }
            if (CONV && !mbar_wait(raw_full(stage), phase, abort_flag, 9u, p.status)) { ok = false; break; }
            tcgen05_fence_after();
            // K-major: rows of 128 B along K (16-byte-chunk swizzle), advance 8 floats = 32 B per MMA.
            // MN-major: one 128-byte row per k (32-byte-chunk swizzle, atoms of four k = 512 B), eight k = 1024 B
            // per MMA, 32-wide column blocks 4096 B apart.
            const uint32_t a_lbo = A_MN ? 4096u : 16u, b_lbo = B_MN ? 4096u : 16u;
            const uint32_t a_sbo = A_MN ? 512u : 1024u, b_sbo = B_MN ? 512u : 1024u;
            const uint32_t a_type = A_MN ? kLayoutSw128Base32 : kLayoutSw128;
            const uint32_t b_type = B_MN ? kLayoutSw128Base32 : kLayoutSw128;
            const uint32_t a_step = A_MN ? 1024u : 32u, b_step = B_MN ? 1024u : 32u;
#pragma unroll
            for (int ks = 0; ks < BK / UMMA_K; ++ks) {
              const uint64_t a_hi = smem_desc(a_main(stage) + ks * a_step, a_lbo, a_sbo, a_type);
              const uint64_t a_sm = smem_desc(a_lo(lo) + ks * a_step, a_lbo, a_sbo, a_type);
              const uint64_t b_hi = smem_desc(b_main(stage) + ks * b_step, b_lbo, b_sbo, b_type);
              const uint64_t b_sm = smem_desc(b_lo(lo) + ks * b_step, b_lbo, b_sbo, b_type);
              umma_tf32(d_tmem, a_sm, b_hi, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);  // small terms first
              umma_tf32(d_tmem, a_hi, b_sm, idesc, 1u);
              umma_tf32(d_tmem, a_hi, b_hi, idesc, 1u);
            }
            umma_commit(stage_free(stage));
            umma_commit(lo_free(lo));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            if (++lo == LO_STAGES) lo = 0;
          }
          if (ok) umma_commit(part_full(part));  // this partial is complete
        }
      }
    }
  }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DRAIN_REGS));
    // ---- drain + epilogue: warps 12..19. Warp w reads TMEM lanes [32*(w%4), +32) and columns [128*h, +128) ----
    const int quad = warp & 3;
    const int half = (warp - 12) >> 2;
    int chunk_index = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn, image_index = 0, z = 0;
      if (CONV) conv_tile_coords(p, tile, tm, tn, image_index); else gemm_tile(tile, tm, tn, z);
      const float alpha = (!CONV && p.alphas) ? p.alphas[z] : p.alpha;
      const float beta = (!CONV && p.betas) ? p.betas[z] : p.beta;
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
        if (lane == 0) mbar_arrive(part_free(part));
      }
      if (!ok) break;
      const int row = tm * BM + quad * 32 + lane;
      const int col0 = tn * BN + half * (BN / 2);
      if (BN == 64 && !CONV && p.c_rowmajor) {  // only the 64-column variant is launched on transposed problems
        if (row < p.m) {
          float* cptr = p.c + z * p.gemm_c_stride + static_cast<long long>(row) * p.ldc + col0;
          if (p.c_vec4 && col0 + BN / 2 <= p.n) {
            float4 old[BN / 8];
            if (use_beta) {  // all old values first: loads and stores through one pointer would serialise
#pragma unroll
              for (int q = 0; q < BN / 8; ++q) old[q] = *reinterpret_cast<const float4*>(cptr + 4 * q);
            }
#pragma unroll
            for (int j = 0; j < BN / 2; j += 4) {
              float4 v;
              v.x = __fmul_rn(alpha, acc[j]); v.y = __fmul_rn(alpha, acc[j + 1]);
              v.z = __fmul_rn(alpha, acc[j + 2]); v.w = __fmul_rn(alpha, acc[j + 3]);
              if (use_beta) {
                v.x = fmaf(beta, old[j / 4].x, v.x); v.y = fmaf(beta, old[j / 4].y, v.y);
                v.z = fmaf(beta, old[j / 4].z, v.z); v.w = fmaf(beta, old[j / 4].w, v.w);
              }
              *reinterpret_cast<float4*>(cptr + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 2; ++j) {
              if (col0 + j < p.n) {
                float v = __fmul_rn(alpha, acc[j]);
                if (use_beta) v = fmaf(beta, cptr[j], v);
                cptr[j] = v;
              }
            }
          }
        }
      } else if (row < p.m) {
        float* cptr = p.c + (CONV ? image_index * p.c_stride : z * p.gemm_c_stride) + static_cast<long long>(col0) * p.ldc + row;
        constexpr int G = 8;
        // G old values are fetched before the first store of a group: loads and stores through one pointer
        // would otherwise be serialised, one memory latency per element.
#pragma unroll
        for (int j0 = 0; j0 < BN / 2; j0 += G) {
          float old[G];
          if (use_beta) {
#pragma unroll
            for (int jj = 0; jj < G; ++jj)
              old[jj] = (col0 + j0 + jj < p.n) ? cptr[static_cast<long long>(j0 + jj) * p.ldc] : 0.f;
          }
#pragma unroll
          for (int jj = 0; jj < G; ++jj) {
            if (col0 + j0 + jj < p.n) {
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
    // ---- split: warps 4..11 turn the raw fp32 tiles into TF32 big parts (in place) and small parts ----
    const int t = threadIdx.x - 4 * 32;  // 0..255
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    if constexpr (MODE == kTma) {
      // Two groups of four warps take alternate K blocks, so the wait / fence / arrive latency of one stage
      // overlaps the conversion work of the next.
      const int group = t >> 7, gt = t & 127;
      constexpr int CHUNKS_ALL = (C::A_BYTES + C::B_BYTES) / 16;
      int kbg = 0;  // running K-block count of this CTA
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kbg) {
          if ((kbg & 1) != group) continue;
          const int st = kbg % STAGES;
          const uint32_t ph = static_cast<uint32_t>(kbg / STAGES) & 1u;
          const int slot = kbg % LO_STAGES;
          ok = mbar_wait(raw_full(st), ph, abort_flag, 5u, p.status);
          // the MMAs of K block kbg - LO_STAGES have read the slot (passes at once on its first use)
          ok = ok && mbar_wait(lo_free(slot), (static_cast<uint32_t>(kbg / LO_STAGES) & 1u) ^ 1u, abort_flag, 7u, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          float4* const main_ptr = reinterpret_cast<float4*>(base_ptr + st * C::MAIN_BYTES);
          float4* const lo_ptr = reinterpret_cast<float4*>(lo_ring + slot * C::MAIN_BYTES);
#pragma unroll 4
          for (int c = gt; c < CHUNKS_ALL; c += 128) {
            const float4 x = main_ptr[c];
            float4 hi, lo;
            hi.x = to_tf32_big(x.x); hi.y = to_tf32_big(x.y); hi.z = to_tf32_big(x.z); hi.w = to_tf32_big(x.w);
            lo.x = to_tf32(x.x - hi.x); lo.y = to_tf32(x.y - hi.y); lo.z = to_tf32(x.z - hi.z);
            lo.w = to_tf32(x.w - hi.w);
            main_ptr[c] = hi;
            lo_ptr[c] = lo;
          }
          fence_proxy_async();  // the tensor cores read these tiles through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(split_full(st));
        }
      }
    } else {
    // Nothing arrives raw in these variants: the split warps write the big and small parts of what they gather
    // (convolution: of op(A) only; both parts of the weights come by TMA).
    // Convolution gather: this thread owns pixel group `pg` (8 consecutive output pixels = one 32-byte swizzle chunk)
    // of the 128-pixel tile and K rows `kr` and `kr + 16` of every K block.
    const int pg = t & 15, kr = t >> 4;
    float gathered[CONV ? 2 : 1][CONV ? 8 : 1];
    // Plain gather: warp `sw` of the eight split warps, lane = position along the contiguous direction, so every
    // load instruction reads one 128-byte run. Sixteen values per operand and K block are held in registers.
    const int sw = t >> 5;
    float ga[GATHER ? 16 : 1], gb[GATHER ? 16 : 1];
    int slot = 0;           // small-part slot of the current K block
    uint32_t slot_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm = 0, tn = 0, image_index = 0;
      const float* image = nullptr;
      int ho0 = 0, wo0 = 0, pixels_left = 0;
      const int khw = CONV ? p.conv.kernel_h * p.conv.kernel_w : 1;
      if (CONV) {
        conv_tile_coords(p, tile, tm, tn, image_index);
        image = p.image + image_index * p.image_stride;
        const int p_first = tm * BM + pg * 8;
        ho0 = p_first / p.conv.out_w;
        wo0 = p_first - ho0 * p.conv.out_w;
        pixels_left = p.m - p_first;  // <= 0: the whole group lies beyond the image
      }
      // Fast gather: what depends on the pixel only is computed once per tile. Eight consecutive pixels of rows that
      // hold at least eight lie on output rows ho0 and ho0 + 1: bit e of row1_mask says which, bit e of live_mask that
      // pixel e exists; pix_off is the pixel's offset inside a channel plane for tap (0, 0) without padding, pix_w its
      // column there.
      int pix_off[CONV ? 8 : 1], pix_w[CONV ? 8 : 1];
      unsigned row1_mask = 0u, live_mask = 0u;
      if (CONV && p.conv_fast) {
        int ho = ho0, wo = wo0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pix_w[e] = wo * p.conv.stride_w;
          pix_off[e] = ho * p.conv.stride_h * p.conv.width + pix_w[e];
          if (ho != ho0) row1_mask |= 1u << e;
          if (e < pixels_left) live_mask |= 1u << e;
          if (++wo == p.conv.out_w) { wo = 0; ++ho; }
        }
      }
      auto gather = [&](int kb) {
        if constexpr (CONV) {
          if (p.conv_fast) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const unsigned kg = static_cast<unsigned>(kb * BK + kr + 16 * u);
              const unsigned c_id = p.khw_magic ? __umulhi(kg, p.khw_magic) : kg;
              const unsigned k2 = kg - c_id * static_cast<unsigned>(khw);
              unsigned kh_id = p.kw_magic ? __umulhi(k2, p.kw_magic) : k2;
              unsigned kw_id = k2 - kh_id * static_cast<unsigned>(p.conv.kernel_w);
              if (p.conv.flip) {
                kh_id = p.conv.kernel_h - 1 - kh_id;
                kw_id = p.conv.kernel_w - 1 - kw_id;
              }
              const int dh = static_cast<int>(kh_id) * p.conv.dil_h - p.conv.pad_h;
              const int dw = static_cast<int>(kw_id) * p.conv.dil_w - p.conv.pad_w;
              const bool row0 = static_cast<unsigned>(ho0 * p.conv.stride_h + dh) < static_cast<unsigned>(p.conv.height);
              const bool row1 =
                  static_cast<unsigned>((ho0 + 1) * p.conv.stride_h + dh) < static_cast<unsigned>(p.conv.height);
              unsigned mask = live_mask & ((row0 ? ~row1_mask : 0u) | (row1 ? row1_mask : 0u));
              if (kg >= static_cast<unsigned>(p.k)) mask = 0u;
              // only formed, never read, where the mask or the column test fails
              const float* base = image + static_cast<long long>(c_id) * p.conv.height * p.conv.width +
                                  (dh * p.conv.width + dw);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const bool ok = ((mask >> e) & 1u) &&
                                static_cast<unsigned>(pix_w[e] + dw) < static_cast<unsigned>(p.conv.width);
                gathered[u][e] = ok ? base[pix_off[e]] : 0.f;
              }
            }
            return;
          }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int kg = kb * BK + kr + 16 * u;
            const int c_id = kg / khw;
            const int k2 = kg - c_id * khw;
            int kh_id = k2 / p.conv.kernel_w;
            int kw_id = k2 - kh_id * p.conv.kernel_w;
            if (p.conv.flip) {
              kh_id = p.conv.kernel_h - 1 - kh_id;
              kw_id = p.conv.kernel_w - 1 - kw_id;
            }
            const float* plane = image + static_cast<long long>(c_id) * p.conv.height * p.conv.width;
            const int dh = kh_id * p.conv.dil_h - p.conv.pad_h, dw = kw_id * p.conv.dil_w - p.conv.pad_w;
            int ho = ho0, wo = wo0;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int hi = ho * p.conv.stride_h + dh, wi = wo * p.conv.stride_w + dw;
              float v = 0.f;
              if (kg < p.k && e < pixels_left && hi >= 0 && hi < p.conv.height && wi >= 0 && wi < p.conv.width)
                v = plane[hi * p.conv.width + wi];
              gathered[u][e] = v;
              if (++wo == p.conv.out_w) { wo = 0; ++ho; }
            }
          }
        }
      };
      int z = 0;
      if (GATHER) gemm_tile(tile, tm, tn, z);
      const float* const a_src = p.a + (p.a_batched ? z * p.a_stride : 0);
      const float* const b_src = p.b + (p.b_batched ? z * p.b_stride : 0);
      // One operand tile of 128 rows x 32 k. MN-contiguous: value j sits at k = sw + 8 (j / 4), row 32 (j % 4) + lane.
      // K-contiguous: value j sits at row sw + 8 j, k = lane.
      auto gather_plain = [&](float (&v)[GATHER ? 16 : 1], const float* src, long long ld, bool mn_major, int row0,
                              int rows_total, int kb) {
        if constexpr (GATHER) {
          if (mn_major) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int kg = kb * BK + sw + 8 * (j >> 2);
              const int row = row0 + 32 * (j & 3) + lane;
              v[j] = (kg < p.k && row < rows_total) ? src[static_cast<long long>(kg) * ld + row] : 0.f;
            }
          } else {
            const int kg = kb * BK + lane;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int row = row0 + sw + 8 * j;
              v[j] = (kg < p.k && row < rows_total) ? src[static_cast<long long>(row) * ld + kg] : 0.f;
            }
          }
        }
      };
      // Writes the sixteen values as TF32 big / small parts at their swizzled positions (conflict-free: the 32 lanes
      // of a warp fill one 128-byte row).
      auto store_plain = [&](const float (&v)[GATHER ? 16 : 1], uint8_t* main_tile, uint8_t* lo_tile, bool mn_major) {
        if constexpr (GATHER) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            int off;
            if (mn_major) {
              const int k = sw + 8 * (j >> 2);
              off = (j & 3) * 4096 + k * 128 + ((((lane >> 3) ^ (k & 3))) << 5) + (lane & 7) * 4;
            } else {
              const int row = sw + 8 * j;
              off = row * 128 + (((lane >> 2) ^ (row & 7)) << 4) + (lane & 3) * 4;
            }
            const float hi = to_tf32_big(v[j]);
            *reinterpret_cast<float*>(main_tile + off) = hi;
            *reinterpret_cast<float*>(lo_tile + off) = to_tf32(v[j] - hi);
          }
        }
      };
      if (CONV) gather(0);
      if (GATHER) {
        gather_plain(ga, a_src, p.lda, A_MN, tm * BM, p.m, 0);
        gather_plain(gb, b_src, p.ldb, B_MN, tn * BN, p.n, 0);
      }
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        // convolution: the stage is ours once its previous MMAs are done (the weights land in it independently and the
        // MMA warp waits for them itself); gathered GEMM: the producer warp forwards "stage free" on raw_full
        ok = CONV ? mbar_wait(stage_free(stage), phase ^ 1u, abort_flag, 5u, p.status)
                  : mbar_wait(raw_full(stage), phase, abort_flag, 5u, p.status);
        ok = ok && mbar_wait(lo_free(slot), slot_phase ^ 1u, abort_flag, 7u, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        float4* const main_ptr = reinterpret_cast<float4*>(base_ptr + stage * C::MAIN_BYTES);
        float4* const lo_ptr = reinterpret_cast<float4*>(lo_ring + slot * C::MAIN_BYTES);
        if constexpr (CONV) {
          // MN-major A tile with the 32-byte-chunk swizzle: column block pg/4 (4096 B each), row k (128 B), chunk
          // (pg % 4) ^ (k % 4) of 32 B holding this thread's eight pixels.
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int k = kr + 16 * u;
            const int f4 = ((pg >> 2) * 4096 + k * 128 + (((pg & 3) ^ (k & 3)) << 5)) >> 4;
            float4 hi0, hi1, lo0, lo1;
            hi0.x = to_tf32_big(gathered[u][0]); hi0.y = to_tf32_big(gathered[u][1]);
            hi0.z = to_tf32_big(gathered[u][2]); hi0.w = to_tf32_big(gathered[u][3]);
            hi1.x = to_tf32_big(gathered[u][4]); hi1.y = to_tf32_big(gathered[u][5]);
            hi1.z = to_tf32_big(gathered[u][6]); hi1.w = to_tf32_big(gathered[u][7]);
            lo0.x = to_tf32(gathered[u][0] - hi0.x); lo0.y = to_tf32(gathered[u][1] - hi0.y);
            lo0.z = to_tf32(gathered[u][2] - hi0.z); lo0.w = to_tf32(gathered[u][3] - hi0.w);
            lo1.x = to_tf32(gathered[u][4] - hi1.x); lo1.y = to_tf32(gathered[u][5] - hi1.y);
            lo1.z = to_tf32(gathered[u][6] - hi1.z); lo1.w = to_tf32(gathered[u][7] - hi1.w);
            main_ptr[f4] = hi0; main_ptr[f4 + 1] = hi1;
            lo_ptr[f4] = lo0; lo_ptr[f4 + 1] = lo1;
          }
          if (kb + 1 < p.k_blocks) gather(kb + 1);  // in flight while B is split and the MMAs run
        }
        if constexpr (GATHER) {
          uint8_t* const stage_ptr = base_ptr + stage * C::MAIN_BYTES;
          uint8_t* const slot_ptr = lo_ring + slot * C::MAIN_BYTES;
          store_plain(ga, stage_ptr, slot_ptr, A_MN);
          store_plain(gb, stage_ptr + C::A_BYTES, slot_ptr + C::A_BYTES, B_MN);
          if (kb + 1 < p.k_blocks) {  // in flight while the tensor cores work on this stage
            gather_plain(ga, a_src, p.lda, A_MN, tm * BM, p.m, kb + 1);
            gather_plain(gb, b_src, p.ldb, B_MN, tn * BN, p.n, kb + 1);
          }
        }
        fence_proxy_async();  // the tensor cores read these tiles through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(split_full(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        if (++slot == LO_STAGES) { slot = 0; slot_phase ^= 1u; }
      }
    }
    }  // gathered / convolution variants
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int MODE = kTma>
cudaError_t launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const Tc32Params& p, int grid,
                           cudaStream_t stream) {
  auto kernel = sgemm_3xtf32_kernel<BN, A_MN, B_MN, MODE>;
  // The kernel re-balances registers between its warpgroups; that only works while the registers the compiler gave
  // each thread at launch cover the budgets it asks for. Refuse (the CUDA-core kernel runs instead) otherwise.
  int regs = 0;
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), Cfg<BN>::SMEM_BYTES, &regs);
  if (e != cudaSuccess) return e;
  if (regs < LAUNCH_REGS) return cudaErrorNotSupported;
  kernel<<<grid, NUM_THREADS, Cfg<BN>::SMEM_BYTES, stream>>>(ma, mb, p);
  return cudaGetLastError();
}

#include "gemm_tc_f32_ts.cuh"

// op(A) through tensor memory (gemm_tc_f32_ts.cuh) unless B200BLAS_SGEMM_TMEM_A=0 asks for the shared-memory kernels.
bool tmem_a_enabled() {
  static const bool on = [] {
    const char* v = std::getenv("B200BLAS_SGEMM_TMEM_A");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return on;
}

template <int BN>
cudaError_t launch_ts(bool a_mn, bool b_mn, const CUtensorMap& ma, const CUtensorMap& mb, const Tc32Params& p, int grid,
                      cudaStream_t stream) {
  if (a_mn) return b_mn ? ts::launch<BN, true, true>(ma, mb, p, grid, stream) : ts::launch<BN, true, false>(ma, mb, p, grid, stream);
  return b_mn ? ts::launch<BN, false, true>(ma, mb, p, grid, stream) : ts::launch<BN, false, false>(ma, mb, p, grid, stream);
}

}  // namespace

cudaError_t launch_tc_f32(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 32 || d.is_conv || d.force_small || d.conj_a || d.conj_b || d.tri) return cudaErrorNotSupported;
  const BatchWalk walk = batch_walk(d);
  if (!walk.ok) return cudaErrorNotSupported;
  // Static selection: the tensor-core path pays off once there are enough 128x256 tiles and K blocks to fill the
  // pipeline; smaller problems keep the k-ascending CUDA-core kernel. B200BLAS_SGEMM=ffma forces the latter.
  static const bool forced_ffma = [] {
    const char* v = std::getenv("B200BLAS_SGEMM");
    return v != nullptr && std::strcmp(v, "ffma") == 0;
  }();
  if (forced_ffma) return cudaErrorNotSupported;
  // one full tile row at least (with op(A) in tensor memory; 256 x 256 for the shared-memory kernels)
  const long long least = tmem_a_enabled() ? 128 : 256;
  if (d.m < least || d.n < least || d.k < 128) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;
  const float* a = static_cast<const float*>(d.a) + d.a_off;
  const float* b = static_cast<const float*>(d.b) + d.b_off;
  // TMA needs 16-byte aligned rows; everything else is gathered with plain loads by the split warps.
  const bool gathered = (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
                        (d.lda % 4) || (d.ldb % 4) || d.lda * 4 >= (1LL << 40) || d.ldb * 4 >= (1LL << 40) ||
                        (walk.a_stride % 4) || (walk.b_stride % 4) || walk.a_stride * 4 >= (1LL << 40) ||
                        walk.b_stride * 4 >= (1LL << 40);

  // From 256^3 multiply-adds on when TMA feeds the kernel (256^3 itself: 40 us on the CUDA-core kernel, whose four
  // tiles leave the machine empty; split along K here), from 512^3 on when the operands have to be gathered.
  const double work = static_cast<double>(d.m) * d.n * d.k * walk.batches;
  if (work < ((gathered || !tmem_a_enabled()) ? 134217728.0 : 16777216.0)) return cudaErrorNotSupported;

  // Tile width: 256 columns amortise the operand traffic best; 128 columns give twice as many tiles and one more
  // pipeline stage, which wins while 256-wide tiles would leave SMs idle.
  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;
  const long long tiles_wide = ((d.m + BM - 1) / BM) * ((d.n + 255) / 256) * walk.batches;
  static const bool forced_128 = [] {  // B200BLAS_SGEMM=single128: no CTA pairs and 128-column tiles whatever the size
    const char* v = std::getenv("B200BLAS_SGEMM");
    return v != nullptr && std::strcmp(v, "single128") == 0;
  }();
  int bn = (!gathered && !forced_128 && tiles_wide >= 2LL * device_sms) ? 256 : 128;
  // Small problems: when twice as many tiles still fit the machine in one wave, 64-column tiles put twice as many
  // SMs to work (1024^3: 64 -> 128 CTAs, 56 -> 66 TFLOP/s).
  const long long tiles_128 = ((d.m + BM - 1) / BM) * ((d.n + 127) / 128) * walk.batches;
  // Better still, with op(A) in tensor memory: keep 128 columns and let the two CTAs of a cluster take half of K each.
  bool split_k = false;
  if (!gathered && bn == 128 && 2 * tiles_128 <= device_sms) {
    static const bool no_split = [] {
      const char* v = std::getenv("B200BLAS_SGEMM_SPLITK");
      return v != nullptr && std::strcmp(v, "0") == 0;
    }();
    split_k = tmem_a_enabled() && !no_split && d.k >= 8 * BK && sm_budget() <= 0;
    if (!split_k) bn = 64;
  }

  CUtensorMap map_a, map_b;
  if (gathered) {
    std::memset(&map_a, 0, sizeof(map_a));
    std::memset(&map_b, 0, sizeof(map_b));
  } else {
    if (!encode_operand_map(&map_a, 4, a, d.m, d.k, d.lda, !d.a_kcontig, BM, walk.a_batches, walk.a_stride))
      return cudaErrorNotSupported;
    if (!encode_operand_map(&map_b, 4, b, d.n, d.k, d.ldb, !d.b_kcontig, bn, walk.b_batches, walk.b_stride))
      return cudaErrorNotSupported;
  }

  Tc32Params p = {};
  p.status = tc_status_device();
  p.a = a; p.b = b;
  p.lda = d.lda; p.ldb = d.ldb;
  p.batches = walk.batches;
  p.a_batched = walk.a_batches > 1;
  p.b_batched = walk.b_batches > 1;
  p.a_stride = walk.a_stride; p.b_stride = walk.b_stride; p.gemm_c_stride = walk.c_stride;
  p.alphas = static_cast<const float*>(d.alphas);
  p.betas = static_cast<const float*>(d.betas);
  p.c = static_cast<float*>(d.c) + d.c_off;
  p.ldc = d.ldc;
  p.m = static_cast<int>(d.m); p.n = static_cast<int>(d.n); p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>((d.m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((d.n + bn - 1) / bn);
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  p.raster_group = 16;

  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * p.batches;
  if (tiles > 0x7FFFFFFF) return cudaErrorNotSupported;
  int sms = device_sms;
  if (sm_budget() > 0 && sm_budget() < sms) sms = sm_budget();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);

  const bool a_mn = !d.a_kcontig, b_mn = !d.b_kcontig;
  if (gathered) {
    *name = "tc_f32_3xtf32_gather_128x128x32";
    if (a_mn) {
      return b_mn ? launch_variant<128, true, true, kGather>(map_a, map_b, p, grid, stream)
                  : launch_variant<128, true, false, kGather>(map_a, map_b, p, grid, stream);
    }
    return b_mn ? launch_variant<128, false, true, kGather>(map_a, map_b, p, grid, stream)
                : launch_variant<128, false, false, kGather>(map_a, map_b, p, grid, stream);
  }
  if (bn == 256) {
    *name = "tc_f32_3xtf32_128x256x32";
    if (a_mn) {
      return b_mn ? launch_variant<256, true, true>(map_a, map_b, p, grid, stream)
                  : launch_variant<256, true, false>(map_a, map_b, p, grid, stream);
    }
    return b_mn ? launch_variant<256, false, true>(map_a, map_b, p, grid, stream)
                : launch_variant<256, false, false>(map_a, map_b, p, grid, stream);
  }
  if (split_k) {
    *name = "tc_f32_3xtf32_128x128x32_splitk2_tmem_a";
    const int t = static_cast<int>(tiles);
    if (a_mn) {
      return b_mn ? ts::launch_splitk<128, true, true>(map_a, map_b, p, t, stream)
                  : ts::launch_splitk<128, true, false>(map_a, map_b, p, t, stream);
    }
    return b_mn ? ts::launch_splitk<128, false, true>(map_a, map_b, p, t, stream)
                : ts::launch_splitk<128, false, false>(map_a, map_b, p, t, stream);
  }
  if (bn != 256 && tmem_a_enabled()) {
    *name = bn == 64 ? "tc_f32_3xtf32_128x64x32_tmem_a" : "tc_f32_3xtf32_128x128x32_tmem_a";
    return bn == 64 ? launch_ts<64>(a_mn, b_mn, map_a, map_b, p, grid, stream)
                    : launch_ts<128>(a_mn, b_mn, map_a, map_b, p, grid, stream);
  }
  if (bn == 64) {
    *name = "tc_f32_3xtf32_128x64x32";
    if (a_mn) {
      return b_mn ? launch_variant<64, true, true>(map_a, map_b, p, grid, stream)
                  : launch_variant<64, true, false>(map_a, map_b, p, grid, stream);
    }
    return b_mn ? launch_variant<64, false, true>(map_a, map_b, p, grid, stream)
                : launch_variant<64, false, false>(map_a, map_b, p, grid, stream);
  }
  *name = "tc_f32_3xtf32_128x128x32";
  if (a_mn) {
    return b_mn ? launch_variant<128, true, true>(map_a, map_b, p, grid, stream)
                : launch_variant<128, true, false>(map_a, map_b, p, grid, stream);
  }
  return b_mn ? launch_variant<128, false, true>(map_a, map_b, p, grid, stream)
              : launch_variant<128, false, false>(map_a, map_b, p, grid, stream);
}

// Batches of problems with at most 64 rows (after layout normalisation) and enough columns to fill a 128-row tile:
// the transposed problem C^T = op(B)^T op(A)^T is computed, one 128 x 64 tile per problem and 128 columns, so the
// narrow dimension becomes the MMA's N. Such batches (2048 x 64x128x96 is the typical one) sit on the FP32 ridge of
// the CUDA cores; on the tensor cores they are bound by HBM traffic alone.
cudaError_t launch_tc_f32_narrow(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 32 || d.is_conv || d.force_small || d.conj_a || d.conj_b || d.tri) return cudaErrorNotSupported;
  static const bool forced_ffma = [] {
    const char* v = std::getenv("B200BLAS_SGEMM");
    return v != nullptr && std::strcmp(v, "ffma") == 0;
  }();
  if (forced_ffma) return cudaErrorNotSupported;
  const BatchWalk walk = batch_walk(d);
  if (!walk.ok) return cudaErrorNotSupported;
  constexpr int BN = 64;
  if (d.m > BN || d.m < 16 || d.n < 64 || d.k < 32 || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;
  const long long tiles = ((d.n + BM - 1) / BM) * walk.batches;
  // A single wide problem of few rows (the 64-row products of the blocked triangular solve: 64 x 8192 x 64 takes 13 us
  // on the CUDA-core kernel) is worth the tensor cores from a quarter of the machine on; batches, which the streaming
  // kernel serves bit-identically to the reference order, only when they fill it.
  const bool single = walk.batches == 1 && tmem_a_enabled();
  if (tiles < (single ? 32 : sm_count()) || tiles > 0x7FFFFFFF) return cudaErrorNotSupported;
  if (static_cast<double>(d.m) * d.n * d.k * walk.batches < (single ? 16777216.0 : 134217728.0)) return cudaErrorNotSupported;
  const float* a = static_cast<const float*>(d.a) + d.a_off;
  const float* b = static_cast<const float*>(d.b) + d.b_off;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (d.lda % 4) || (d.ldb % 4) ||
      (walk.a_stride % 4) || (walk.b_stride % 4))
    return cudaErrorNotSupported;

  // operands swapped: the kernel's A (128-row tiles) is op(B)^T, its B (64 columns) is op(A)^T
  CUtensorMap map_a, map_b;
  if (!encode_operand_map(&map_a, 4, b, d.n, d.k, d.ldb, !d.b_kcontig, BM, walk.b_batches, walk.b_stride))
    return cudaErrorNotSupported;
  if (!encode_operand_map(&map_b, 4, a, d.m, d.k, d.lda, !d.a_kcontig, BN, walk.a_batches, walk.a_stride))
    return cudaErrorNotSupported;

  Tc32Params p = {};
  p.status = tc_status_device();
  p.c = static_cast<float*>(d.c) + d.c_off;
  p.ldc = d.ldc;
  p.m = static_cast<int>(d.n); p.n = static_cast<int>(d.m); p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>((d.n + BM - 1) / BM);
  p.tiles_n = 1;
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  p.raster_group = 16;
  p.batches = walk.batches;
  p.a_batched = walk.b_batches > 1;
  p.b_batched = walk.a_batches > 1;
  p.gemm_c_stride = walk.c_stride;
  p.alphas = static_cast<const float*>(d.alphas);
  p.betas = static_cast<const float*>(d.betas);
  p.c_rowmajor = 1;
  p.c_vec4 = ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0 && d.ldc % 4 == 0 && walk.c_stride % 4 == 0) ? 1 : 0;

  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;
  int sms = device_sms;
  if (sm_budget() > 0 && sm_budget() < sms) sms = sm_budget();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  const bool a_mn = !d.b_kcontig, b_mn = !d.a_kcontig;
  if (tmem_a_enabled()) {
    *name = "tc_f32_3xtf32_narrow_128x64x32_tmem_a";
    return launch_ts<BN>(a_mn, b_mn, map_a, map_b, p, grid, stream);
  }
  *name = "tc_f32_3xtf32_narrow_128x64x32";
  if (a_mn) {
    return b_mn ? launch_variant<BN, true, true>(map_a, map_b, p, grid, stream)
                : launch_variant<BN, true, false>(map_a, map_b, p, grid, stream);
  }
  return b_mn ? launch_variant<BN, false, true>(map_a, map_b, p, grid, stream)
              : launch_variant<BN, false, false>(map_a, map_b, p, grid, stream);
}

namespace {
// Big and small TF32 parts of the weights [rows][k] (leading dimension ld) into two planes with pitch `pitch`.
__global__ void split_weights_kernel(const float* __restrict__ w, long long ld, int rows, int k, int pitch,
                                     float* __restrict__ big, float* __restrict__ small) {
  const long long total = static_cast<long long>(rows) * pitch;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / pitch), c = static_cast<int>(i - static_cast<long long>(r) * pitch);
    const float x = c < k ? w[r * ld + c] : 0.f;
    const float hi = tc::to_tf32_big(x);
    big[i] = hi;
    small[i] = tc::to_tf32(x - hi);
  }
}
}  // namespace

cudaError_t launch_tc_conv_f32(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 32 || !d.is_conv) return cudaErrorNotSupported;
  static const bool forced_ffma = [] {
    const char* v = std::getenv("B200BLAS_SGEMM");
    return v != nullptr && std::strcmp(v, "ffma") == 0;
  }();
  if (forced_ffma) return cudaErrorNotSupported;
  const float* weights = static_cast<const float*>(d.b) + d.b_off;
  if (d.m > 0x7FFFFFFF || d.n > 0x7FFFFFFF || d.k > 0x7FFFFFFF || d.batch > 0x7FFFFFFF) return cudaErrorNotSupported;
  constexpr int BN = 128;
  const long long tiles = ((d.m + BM - 1) / BM) * ((d.n + BN - 1) / BN) * d.batch;
  if (d.m < 128 || d.n < 32 || d.k < 64 || tiles < 64 || tiles > 0x7FFFFFFF) return cudaErrorNotSupported;

  // The weights [Cout][K] are the K-major B operand of every tile of every image: they are split once into two planes
  // of stream-ordered scratch (pitch rounded up to 16 bytes, so any K and any alignment of the caller's buffer will
  // do), and both planes travel by TMA.
  const long long pitch = (d.k + 3) / 4 * 4;
  const size_t plane_bytes = (static_cast<size_t>(d.n) * pitch * 4 + 255) / 256 * 256;
  float* planes = nullptr;
  cudaError_t err = cudaMallocAsync(reinterpret_cast<void**>(&planes), 2 * plane_bytes, stream);
  if (err != cudaSuccess) return err;
  float* const small_plane = planes + plane_bytes / 4;
  struct Release {  // stream-ordered: the kernels enqueued below still see the planes
    float* ptr; cudaStream_t stream;
    ~Release() { cudaFreeAsync(ptr, stream); }
  } release{planes, stream};
  CUtensorMap map_b, map_small;
  if (!encode_operand_map(&map_b, 4, planes, d.n, d.k, pitch, false, BN, 1, 0)) return cudaErrorNotSupported;
  if (!encode_operand_map(&map_small, 4, small_plane, d.n, d.k, pitch, false, BN, 1, 0)) return cudaErrorNotSupported;
  {
    const long long total = d.n * pitch;
    const unsigned blocks = static_cast<unsigned>(total / 256 + 1 < 4096 ? total / 256 + 1 : 4096);
    split_weights_kernel<<<blocks, 256, 0, stream>>>(weights, d.ldb, static_cast<int>(d.n), static_cast<int>(d.k),
                                                     static_cast<int>(pitch), planes, small_plane);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }

  Tc32Params p = {};
  p.status = tc_status_device();
  p.c = static_cast<float*>(d.c) + d.c_off;
  p.ldc = d.ldc;
  p.m = static_cast<int>(d.m); p.n = static_cast<int>(d.n); p.k = static_cast<int>(d.k);
  p.tiles_m = static_cast<int>((d.m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((d.n + BN - 1) / BN);
  p.k_blocks = static_cast<int>((d.k + BK - 1) / BK);
  p.alpha = 1.f;
  p.beta = 0.f;
  p.raster_group = 16;
  p.image = static_cast<const float*>(d.a) + d.a_off;
  p.image_stride = d.a_stride;
  p.c_stride = d.c_stride;
  p.batch = static_cast<int>(d.batch);
  p.conv = d.conv;
  {
    const long long khw = static_cast<long long>(d.conv.kernel_h) * d.conv.kernel_w;
    const long long span = (static_cast<long long>(d.conv.height) + 2LL * (d.conv.pad_h > 0 ? d.conv.pad_h : 0) +
                            d.conv.stride_h + static_cast<long long>(d.conv.kernel_h) * d.conv.dil_h) *
                               d.conv.width +
                           static_cast<long long>(d.conv.kernel_w) * d.conv.dil_w + d.conv.pad_w;
    static const bool slow_gather = [] {
      const char* v = std::getenv("B200BLAS_CONV_GATHER");
      return v != nullptr && std::strcmp(v, "general") == 0;
    }();
    // multiply-high by ceil(2^32 / d) equals the quotient while dividend * d < 2^32
    p.conv_fast = !slow_gather && d.conv.out_w >= 8 && (d.k + 64) * khw < (1LL << 32) && khw * d.conv.kernel_w < (1LL << 32) &&
                  span < (1LL << 31) && d.conv.stride_h > 0 && d.conv.stride_w > 0;
    p.khw_magic = khw > 1 ? static_cast<unsigned>(((1ULL << 32) + khw - 1) / khw) : 0u;
    p.kw_magic = d.conv.kernel_w > 1 ? static_cast<unsigned>(((1ULL << 32) + d.conv.kernel_w - 1) / d.conv.kernel_w) : 0u;
  }

  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;
  int sms = device_sms;
  if (sm_budget() > 0 && sm_budget() < sms) sms = sm_budget();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  // The tensor-memory kernel addresses the image with 32-bit offsets and keeps a table of the K rows in shared memory.
  const long long image_span = (static_cast<long long>(d.conv.channels) * d.conv.height +
                                static_cast<long long>(d.conv.kernel_h) * d.conv.dil_h + d.conv.pad_h + d.conv.stride_h) *
                                   d.conv.width + static_cast<long long>(d.conv.kernel_w) * d.conv.dil_w;
  const bool taps_fit = d.conv.height < 0x7000 && d.conv.width < 0x7000 && d.conv.pad_h < 0x800 &&
                        static_cast<long long>(d.conv.kernel_h) * d.conv.dil_h < 0x7000 &&
                        static_cast<long long>(d.conv.kernel_w) * d.conv.dil_w < 0x7000;
  if (tmem_a_enabled() && taps_fit && image_span < 0x20000000LL && ts::smem_bytes<BN, true>(p) <= 227 * 1024) {
    *name = "tc_conv_f32_3xtf32_128x128x32_tmem_a";
    return ts::launch<BN, false, false, true>(map_small, map_b, p, grid, stream);
  }
  *name = "tc_conv_f32_3xtf32_128x128x32";
  return launch_variant<BN, true, false, kConv>(map_small, map_b, p, grid, stream);
}

}  // namespace b200
