// 3xTF32 SGEMM / Convgemm with op(A) in tensor memory (included by gemm_tc_f32.cu, which defines Tc32Params, the tile
// numbering and the constants used here).
//
// The kernel in gemm_tc_f32.cu keeps both TF32 parts of both operands in shared memory, and with 128-row tiles on one
// SM that memory's bandwidth is the limit: per K block of a 128 x 64 tile it moves 24 KB in by TMA, 72 KB through the
// split warps and 72 KB into the tensor cores (a timeline of 1024^3 shows 0.67 us per K block = 168 KB at 128 B per
// clock, with the tensor pipe 17 % busy). tcgen05.mma can take its A operand from tensor memory instead: here the
// split warps write the big and small parts of op(A) with tcgen05.st into TMEM columns next to the accumulators (lane =
// row of the tile, column = k), so op(A) is read from shared memory once (the raw tile) and never written back, and
// the MMAs read only op(B) from shared memory: 88 KB per K block instead of 168 (128 x 128 tiles: 144 instead of 224).
// For convolutions op(A) never touches shared memory at all: each split thread owns one output pixel (= one TMEM lane),
// gathers its 16 taps of the K block from the image (consecutive lanes = consecutive pixels, so the loads coalesce;
// what a K row means - channel plane, tap row and column - is decoded once per launch into a table in shared memory)
// and stores both parts to TMEM; both parts of the weights arrive by TMA.
//
// Arithmetic, chunked accumulation, roles and register budgets are those of gemm_tc_f32.cu: x = hi + lo,
// lo_a*hi_b + hi_a*lo_b + hi_a*hi_b accumulated over 128 K in one of two TMEM partials that the drain warps add into
// fp32 registers. Results are bit-identical to that kernel's.
//
// TMEM columns: [0, 2 BN) the two partials, then LO_STAGES slots of 64 columns (32 big + 32 small parts of a K block).

namespace ts {

template <int BN, bool CONV>
struct Cfg {
  static constexpr int A_BYTES = CONV ? 0 : BM * BK * 4;  // raw op(A) tile; the convolution gathers it
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int MAIN_BYTES = A_BYTES + B_BYTES;     // one K block as TMA delivers it (B becomes its big part)
  static constexpr int LO_BYTES = B_BYTES;                 // small part of B
  static constexpr int LO_STAGES = (BN == 64) ? 4 : 3;
  static constexpr int STAGES = CONV ? 4 : (BN == 64) ? 6 : 5;
  static constexpr int SMEM_BYTES = STAGES * MAIN_BYTES + LO_STAGES * LO_BYTES + 1024 + 512;  // + the tap table (CONV)
  static constexpr int A_COLS = 2 * BN;                    // first TMEM column of the op(A) slots
  static_assert(A_COLS + 64 * LO_STAGES <= TMEM_COLS, "tensor memory columns");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
};

__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Eight consecutive 32-bit columns of the calling thread's TMEM lane.
__device__ __forceinline__ void tmem_st_8cols(uint32_t taddr, const float (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
               "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Splits eight values and stores the big parts at `big_col`, the small parts 32 columns further.
__device__ __forceinline__ void split_store_8(uint32_t big_col, const float (&x)[8]) {
  float hi[8], lo[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    hi[i] = to_tf32_big(x[i]);
    lo[i] = to_tf32(x[i] - hi[i]);
  }
  tmem_st_8cols(big_col, hi);
  tmem_st_8cols(big_col + 32u, lo);
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
  return v;
}

// SPLITK: launched as clusters of two CTAs with exactly one tile per cluster; CTA r of the cluster multiplies the r-th
// half of K, CTA 1 hands its sums to CTA 0 through distributed shared memory, CTA 0 adds them and writes C. For
// problems with so few tiles that half the SMs would idle (1024^3: 64 tiles of 128 x 128 on 128 SMs, each with half
// as many K blocks as a 128 x 64 tile would need, and MMAs twice as wide for little more issue time).
template <int BN, bool A_MN, bool B_MN, bool CONV, bool SPLITK = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
sgemm_3xtf32_ts_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const Tc32Params p) {
  using C = Cfg<BN, CONV>;
  constexpr int STAGES = C::STAGES;
  constexpr int LO_STAGES = C::LO_STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  uint8_t* const base_ptr = smem_raw + (tiles_base - raw);
  uint8_t* const lo_ring = base_ptr + STAGES * C::MAIN_BYTES;
  uint64_t* const bars = reinterpret_cast<uint64_t*>(lo_ring + LO_STAGES * C::LO_BYTES);
  const uint32_t bar_base = smem_u32(bars);
  // [0,S) TMA data landed, [S,2S) split done, [2S,3S) stage free, 2 partial-full, 2 partial-free, L slot free
  auto raw_full = [&](int s) { return bar_base + 8u * s; };
  auto split_full = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto stage_free = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto part_full = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
  auto part_free = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
  auto lo_free = [&](int l) { return bar_base + 8u * (3 * STAGES + 4 + l); };
  uint32_t* const tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4 + LO_STAGES);
  static_assert((3 * STAGES + 4 + LO_STAGES) * 8 + 8 <= 512, "barrier block");
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  // broadcast from lane 0: tells the compiler the value is the same for the whole warp, so everything derived from
  // it (roles, K rows, the decoded tap of the convolution) stays in uniform registers
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * (CONV ? p.batch : p.batches);
  auto gemm_tile = [&](int tile, int& tm, int& tn, int& z) {
    z = tile / tiles_per_problem;
    tile_coords(p, tile - z * tiles_per_problem, tm, tn);
  };
  static_assert(!(SPLITK && CONV), "the convolution is not split along K");
  const int crank = SPLITK ? static_cast<int>(cluster_ctarank()) : 0;
  const int first_tile = SPLITK ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = SPLITK ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // this CTA's share of the K blocks
  const int kb_half = (p.k_blocks + 1) / 2;
  const int kb_begin = SPLITK ? crank * kb_half : 0;
  const int kb_count = SPLITK ? min(kb_half, p.k_blocks - kb_begin) : p.k_blocks;
  constexpr int SPLIT_REGS = CONV ? 112 : 72;  // the convolution keeps 32 gathered values in flight
  constexpr int DRAIN_REGS = CONV ? 104 : 136;
  static_assert(BN <= 128, "the drain warps hold BN / 2 accumulators in 136 registers");
  static_assert(128 * 40 + 256 * SPLIT_REGS + 256 * DRAIN_REGS <= NUM_THREADS * LAUNCH_REGS, "register budgets");

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(raw_full(s), 1);
      mbar_init(split_full(s), 4);  // one arrival per warp of the group that splits the stage
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
  // Convolution: one entry per K row of the padded K extent, {offset of tap (kh, kw) of channel c from the pixel's
  // own offset, (kh * dilation) << 16 | kw * dilation}; rows beyond K get a tap row that is outside every image (the
  // launcher only takes images of fewer than 0x7000 rows).
  int2* const tap_table = reinterpret_cast<int2*>(reinterpret_cast<uint8_t*>(bars) + 512);
  if constexpr (CONV) {
    const int khw = p.conv.kernel_h * p.conv.kernel_w;
    for (int kg = threadIdx.x; kg < p.k_blocks * BK; kg += NUM_THREADS) {
      int2 e = make_int2(0, 0x7FFF0000);  // outside for live pixels and for the marker of dead ones alike
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
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // shared memory: STAGES x (A raw | B main), then LO_STAGES x B small; K block g uses stage g % STAGES, slot g % LO_STAGES
  auto a_main = [&](int s) { return tiles_base + s * C::MAIN_BYTES; };
  auto b_main = [&](int s) { return a_main(s) + C::A_BYTES; };
  auto b_lo = [&](int l) { return tiles_base + STAGES * C::MAIN_BYTES + l * C::LO_BYTES; };
  auto a_cols = [&](int l) { return static_cast<uint32_t>(C::A_COLS + 64 * l); };  // big parts; small parts 32 further

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ---- TMA producer ----
      if (lane == 0) {
        int stage = 0, slot = 0, issued = 0;
        uint32_t phase = 0, slot_phase = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
          int tm, tn, image_index = 0, z = 0;
          if (CONV) conv_tile_coords(p, tile, tm, tn, image_index); else gemm_tile(tile, tm, tn, z);
          const int az = p.a_batched ? z : 0, bz = p.b_batched ? z : 0;
          for (int kb = 0; kb < kb_count; ++kb) {
            if (!mbar_wait(stage_free(stage), phase ^ 1u, abort_flag, 1u, p.status)) { ok = false; break; }
            if (CONV) {
              // both parts of the weights were prepared once for all tiles: map_b the big parts, map_a the small ones
              if (!mbar_wait(lo_free(slot), slot_phase ^ 1u, abort_flag, 8u, p.status)) { ok = false; break; }
              mbar_arrive_expect_tx(raw_full(stage), 2 * C::B_BYTES);
              tma_load_3d(b_main(stage), &map_b, raw_full(stage), kb * BK, tn * BN, 0);
              tma_load_3d(b_lo(slot), &map_a, raw_full(stage), kb * BK, tn * BN, 0);
              if (++slot == LO_STAGES) { slot = 0; slot_phase ^= 1u; }
            } else {
              mbar_arrive_expect_tx(raw_full(stage), C::A_BYTES + C::B_BYTES);
              if (A_MN) {
#pragma unroll
                for (int j = 0; j < BM / 32; ++j)
                  tma_load_3d(a_main(stage) + j * 4096, &map_a, raw_full(stage), tm * BM + j * 32, (kb_begin + kb) * BK, az);
              } else {
                tma_load_3d(a_main(stage), &map_a, raw_full(stage), (kb_begin + kb) * BK, tm * BM, az);
              }
              if (B_MN) {
#pragma unroll
                for (int j = 0; j < BN / 32; ++j)
                  tma_load_3d(b_main(stage) + j * 4096, &map_b, raw_full(stage), tn * BN + j * 32, (kb_begin + kb) * BK, bz);
              } else {
                tma_load_3d(b_main(stage), &map_b, raw_full(stage), (kb_begin + kb) * BK, tn * BN, bz);
              }
            }
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
            while (!mbar_try_wait(raw_full(s), par) && clock64() - start < kWaitCycles / 8) {}
          }
        }
      }
    } else if (warp == 1) {
      // ---- MMA issuer: op(A) from tensor memory (K-major by construction), op(B) from shared memory ----
      if (lane == 0) {
        constexpr uint32_t idesc = make_idesc(BM, BN, 2, 0, B_MN ? 1 : 0);
        int stage = 0, lo = 0, chunk_index = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
          for (int kb0 = 0; kb0 < kb_count && ok; kb0 += CHUNK_KB, ++chunk_index) {
            const int part = chunk_index & 1;
            const uint32_t part_phase = (chunk_index >> 1) & 1u;
            if (!mbar_wait(part_free(part), part_phase ^ 1u, abort_flag, 2u, p.status)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(part * BN);
            const int kb_end = min(kb0 + CHUNK_KB, kb_count);
            for (int kb = kb0; kb < kb_end; ++kb) {
              if (!mbar_wait(split_full(stage), phase, abort_flag, 3u, p.status)) { ok = false; break; }
              if (CONV && !mbar_wait(raw_full(stage), phase, abort_flag, 9u, p.status)) { ok = false; break; }
              tcgen05_fence_after();
              const uint32_t b_lbo = B_MN ? 4096u : 16u, b_sbo = B_MN ? 512u : 1024u;
              const uint32_t b_type = B_MN ? kLayoutSw128Base32 : kLayoutSw128;
              const uint32_t b_step = B_MN ? 1024u : 32u;
              const uint32_t a_big = tmem_base + a_cols(lo), a_small = a_big + 32u;
#pragma unroll
              for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                const uint64_t b_hi = smem_desc(b_main(stage) + ks * b_step, b_lbo, b_sbo, b_type);
                const uint64_t b_sm = smem_desc(b_lo(lo) + ks * b_step, b_lbo, b_sbo, b_type);
                umma_tf32_ts(d_tmem, a_small + ks * UMMA_K, b_hi, idesc, (kb != kb0 || ks != 0) ? 1u : 0u);
                umma_tf32_ts(d_tmem, a_big + ks * UMMA_K, b_sm, idesc, 1u);
                umma_tf32_ts(d_tmem, a_big + ks * UMMA_K, b_hi, idesc, 1u);
              }
              umma_commit(stage_free(stage));
              umma_commit(lo_free(lo));
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
              if (++lo == LO_STAGES) lo = 0;
            }
            if (ok) umma_commit(part_full(part));
          }
        }
      }
    }
  } else if (warp >= 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(DRAIN_REGS));
    // ---- drain + epilogue: warp w reads TMEM lanes [32 (w % 4), +32), columns [BN/2 * h, +BN/2) of each partial ----
    const int quad = warp & 3;
    const int half = (warp - 12) >> 2;
    int chunk_index = 0;
    int cluster_syncs = 0;  // SPLITK: every thread of the cluster passes the cluster barrier exactly twice
    bool ok = true;
    for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
      int tm, tn, image_index = 0, z = 0;
      if (CONV) conv_tile_coords(p, tile, tm, tn, image_index); else gemm_tile(tile, tm, tn, z);
      const float alpha = (!CONV && p.alphas) ? p.alphas[z] : p.alpha;
      const float beta = (!CONV && p.betas) ? p.betas[z] : p.beta;
      const bool use_beta = beta != 0.f;
      float acc[BN / 2];
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) acc[j] = 0.f;
      for (int kb0 = 0; kb0 < kb_count; kb0 += CHUNK_KB, ++chunk_index) {
        const int part = chunk_index & 1;
        const uint32_t part_phase = (chunk_index >> 1) & 1u;
        ok = mbar_wait(part_full(part), part_phase, abort_flag, 4u, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               static_cast<uint32_t>(part * BN + half * (BN / 2));
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
      if constexpr (SPLITK) {
        // The rings are idle now (every load has landed, every MMA has read its operands): CTA 1 leaves its sums in
        // its own shared memory, [column][thread] so that neither side has bank conflicts, and CTA 0 fetches them.
        float* const scratch = reinterpret_cast<float*>(base_ptr);
        const int dt = static_cast<int>(threadIdx.x) - 12 * 32;
        if (crank == 1) {
#pragma unroll
          for (int j = 0; j < BN / 2; ++j) scratch[j * 256 + dt] = acc[j];
        }
        cluster_sync_all();
        if (crank == 0) {
          const uint32_t peer = map_to_cta(smem_u32(scratch), 1u);
#pragma unroll
          for (int j = 0; j < BN / 2; ++j) acc[j] += ld_cluster_f32(peer + static_cast<uint32_t>(j * 256 + dt) * 4u);
        }
        cluster_sync_all();  // CTA 1 stays until its memory has been read
        cluster_syncs = 2;
        if (crank != 0) continue;
      }
      const int row = tm * BM + quad * 32 + lane;
      const int col0 = tn * BN + half * (BN / 2);
      if (BN == 64 && !CONV && p.c_rowmajor) {  // transposed problems: a thread's results are contiguous in memory
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
        float* cptr = p.c + (CONV ? image_index * p.c_stride : z * p.gemm_c_stride) +
                      static_cast<long long>(col0) * p.ldc + row;
        constexpr int G = 8;  // old values of a group are fetched before its first store (see gemm_tc_f32.cu)
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
    if constexpr (SPLITK) {
      for (; cluster_syncs < 2; ++cluster_syncs) cluster_sync_all();  // a role that gave up still meets its peer
    }
  } else {
    if constexpr (SPLIT_REGS > LAUNCH_REGS) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SPLIT_REGS));
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(SPLIT_REGS));
    }
    // ---- split: warps 4..11. Warp w owns TMEM lanes [32 (w % 4), +32), i.e. rows 32 (w % 4) + lane of the tile ----
    const int t = threadIdx.x - 4 * 32;  // 0..255
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    bool ok = true;
    if constexpr (!CONV) {
      // Two groups of four warps (one warp per lane quadrant each) take alternate K blocks.
      const int group = t >> 7, gt = t & 127;
      constexpr int B_CHUNKS = C::B_BYTES / 16;
      int kbg = 0;  // running K-block count of this CTA
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        for (int kb = 0; kb < kb_count; ++kb, ++kbg) {
          if ((kbg & 1) != group) continue;
          const int st = kbg % STAGES;
          const uint32_t ph = static_cast<uint32_t>(kbg / STAGES) & 1u;
          const int slot = kbg % LO_STAGES;
          ok = mbar_wait(raw_full(st), ph, abort_flag, 5u, p.status);
          // the MMAs of K block kbg - LO_STAGES have read the slot (passes at once on its first use)
          ok = ok && mbar_wait(lo_free(slot), (static_cast<uint32_t>(kbg / LO_STAGES) & 1u) ^ 1u, abort_flag, 7u, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tcgen05_fence_after();
          const uint8_t* const a_tile = base_ptr + st * C::MAIN_BYTES;
          const uint32_t big0 = lane_base + a_cols(slot);
#pragma unroll
          for (int b8 = 0; b8 < BK / 8; ++b8) {
            float x[8];
            if (A_MN) {
              // [k][m] rows of 128 B per 32-wide block of m (block = this warp's quadrant), 32-byte-chunk swizzle
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int k = b8 * 8 + i;
                x[i] = *reinterpret_cast<const float*>(a_tile + quad * 4096 + k * 128 + ((((lane >> 3) ^ (k & 3))) << 5) +
                                                       (lane & 7) * 4);
              }
            } else {
              // [m][k] rows of 128 B, 16-byte-chunk swizzle
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int chunk = b8 * 2 + h;
                const float4 v = *reinterpret_cast<const float4*>(a_tile + row_in_tile * 128 +
                                                                  ((chunk ^ (row_in_tile & 7)) << 4));
                x[4 * h] = v.x; x[4 * h + 1] = v.y; x[4 * h + 2] = v.z; x[4 * h + 3] = v.w;
              }
            }
            split_store_8(big0 + b8 * 8, x);
          }
          float4* const b_ptr = reinterpret_cast<float4*>(base_ptr + st * C::MAIN_BYTES + C::A_BYTES);
          float4* const b_small = reinterpret_cast<float4*>(lo_ring + slot * C::LO_BYTES);
#pragma unroll 4
          for (int c = gt; c < B_CHUNKS; c += 128) {
            const float4 x = b_ptr[c];
            float4 hi, lo;
            hi.x = to_tf32_big(x.x); hi.y = to_tf32_big(x.y); hi.z = to_tf32_big(x.z); hi.w = to_tf32_big(x.w);
            lo.x = to_tf32(x.x - hi.x); lo.y = to_tf32(x.y - hi.y); lo.z = to_tf32(x.z - hi.z);
            lo.w = to_tf32(x.w - hi.w);
            b_ptr[c] = hi;
            b_small[c] = lo;
          }
          tmem_st_wait();
          fence_proxy_async();  // shared memory written above is read by the tensor cores through the async proxy
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(split_full(st));
        }
      }
    } else {
      // Convolution: as above, two groups of four warps take alternate K blocks. A thread gathers the 32 taps of its
      // pixel for the group's NEXT K block (two K blocks ahead in the CTA's order, also across a tile boundary) before
      // it waits on anything, so the loads have two K-block periods to come back.
      const int group = t >> 7;
      float g[32];
      // where the gather stands: tile, K block, and what depends on the tile's pixel
      int g_tile = blockIdx.x, g_kb = group;
      const float* g_image = nullptr;
      int g_h0 = 0, g_w0 = 0, g_off = 0;
      auto enter_tile = [&]() {
        int tm, tn, image_index;
        conv_tile_coords(p, g_tile, tm, tn, image_index);
        g_image = p.image + image_index * p.image_stride;
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
        for (int j0 = 0; j0 < 32; j0 += 8) {
#pragma unroll
          for (int j = j0; j < j0 + 8; ++j) {
            const int2 e = taps[j];  // the same address for every lane: one broadcast read
            const bool inside = static_cast<unsigned>(g_h0 + (e.y >> 16)) < static_cast<unsigned>(p.conv.height) &&
                                static_cast<unsigned>(g_w0 + (e.y & 0xFFFF)) < static_cast<unsigned>(p.conv.width);
            g[j] = inside ? g_image[e.x + g_off] : 0.f;
          }
          asm volatile("" ::: "memory");  // eight table entries at a time: all 32 at once would not fit the registers
        }
      };
      // the group's next K block: two further in the CTA's running order (a tile has at least two K blocks)
      auto advance = [&]() {
        g_kb += 2;
        if (g_kb >= p.k_blocks) {
          g_kb -= p.k_blocks;
          g_tile += gridDim.x;
          if (g_tile < num_tiles) enter_tile();
        }
      };
      if (g_kb >= p.k_blocks) {  // cannot happen while tiles have two K blocks or more; keeps the walk well-defined
        g_kb -= p.k_blocks;
        g_tile += gridDim.x;
      }
      if (g_tile < num_tiles) {
        enter_tile();
        gather();
      }
      int kbg = 0;  // running K-block count of this CTA
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++kbg) {
          if ((kbg & 1) != group) continue;
          const int st = kbg % STAGES;
          const int slot = kbg % LO_STAGES;
          ok = mbar_wait(lo_free(slot), (static_cast<uint32_t>(kbg / LO_STAGES) & 1u) ^ 1u, abort_flag, 7u, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t big0 = lane_base + a_cols(slot);
#pragma unroll
          for (int b8 = 0; b8 < BK / 8; ++b8) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = g[b8 * 8 + i];
            split_store_8(big0 + b8 * 8, x);
          }
          advance();
          if (g_tile < num_tiles) gather();  // in flight while the stores complete and the MMAs run
          tmem_st_wait();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(split_full(st));
        }
      }
    }
  }

  if constexpr (SPLITK) {
    if (warp < 12) {  // the drain warps have passed them where they exchange the sums
      __syncwarp();
      cluster_sync_all();
      cluster_sync_all();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Shared memory of one launch: the rings and, for a convolution, 8 bytes per K row of the padded K extent.
template <int BN, bool CONV>
long long smem_bytes(const Tc32Params& p) {
  return Cfg<BN, CONV>::SMEM_BYTES + (CONV ? 8LL * p.k_blocks * BK : 0LL);
}

// Split-K launch: `tiles` clusters of two CTAs.
template <int BN, bool A_MN, bool B_MN>
cudaError_t launch_splitk(const CUtensorMap& ma, const CUtensorMap& mb, const Tc32Params& p, int tiles,
                          cudaStream_t stream) {
  auto kernel = sgemm_3xtf32_ts_kernel<BN, A_MN, B_MN, false, true>;
  constexpr int smem = Cfg<BN, false>::SMEM_BYTES;
  static_assert(256 * (BN / 2) * 4 <= Cfg<BN, false>::STAGES * Cfg<BN, false>::MAIN_BYTES, "exchange area");
  int regs = 0;
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), smem, &regs);
  if (e != cudaSuccess) return e;
  if (regs < LAUNCH_REGS) return cudaErrorNotSupported;  // the register re-balancing needs the full pool
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(2 * tiles));
  config.blockDim = dim3(NUM_THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute cluster;
  cluster.id = cudaLaunchAttributeClusterDimension;
  cluster.val.clusterDim.x = 2;
  cluster.val.clusterDim.y = 1;
  cluster.val.clusterDim.z = 1;
  config.attrs = &cluster;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, ma, mb, p);
}

template <int BN, bool A_MN, bool B_MN, bool CONV = false>
cudaError_t launch(const CUtensorMap& ma, const CUtensorMap& mb, const Tc32Params& p, int grid, cudaStream_t stream) {
  auto kernel = sgemm_3xtf32_ts_kernel<BN, A_MN, B_MN, CONV>;
  const long long smem = smem_bytes<BN, CONV>(p);
  if (smem > 227 * 1024) return cudaErrorNotSupported;
  int regs = 0;
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), static_cast<int>(smem), &regs);
  if (e != cudaSuccess) return e;
  if (regs < LAUNCH_REGS) return cudaErrorNotSupported;  // the register re-balancing needs the full pool
  kernel<<<grid, NUM_THREADS, static_cast<size_t>(smem), stream>>>(ma, mb, p);
  return cudaGetLastError();
}

}  // namespace ts
