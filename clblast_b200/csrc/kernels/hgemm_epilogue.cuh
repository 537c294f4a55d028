// Epilogue of the half-precision tensor-core kernels: alpha * acc (+ beta * c) in fp32, one rounding to half, and
// the way out of the SM.
//
// Four epilogue warps own the 128 accumulator rows of a CTA; a thread holds 32 consecutive columns of one row, while
// C is contiguous along the rows. Writing those values with one 2-byte store per element costs ~11 us per
// 128 x 256 tile (measured: 155 us for an 8192 x 8192 result whatever K is). Instead each 128 x 32 block is put
// into shared memory column by column ([column][128 rows], 256 bytes per column) and one thread hands it to the
// TMA unit, which writes whole lines, clips the block at the edges of C and runs while the warps convert the next
// block. Four staging buffers rotate, so one named barrier per block orders everything: after issuing the store
// of block s the elected thread waits until the store of block s - 2 has left its buffer (`wait_group.read 2`);
// it then passes the barrier of block s + 1, and only after that barrier do the warps write block s + 2 into that
// very buffer.
//
// The TMA path needs C 16-byte aligned with a leading dimension (and batch stride) that is a multiple of 8
// elements; otherwise the values go out with plain stores. With beta != 0 the old block is fetched into the same
// staging buffer by a TMA load two blocks ahead (the first two of a tile before the accumulator is even waited for)
// and combined in place.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "tc_common.cuh"

namespace b200 {
namespace tc {

constexpr int kStageRows = 128;                                  // rows of C per CTA
constexpr int kStageCols = 32;                                   // columns per staged block
constexpr int kStageBytes = kStageRows * kStageCols * 2;         // 8 KB
constexpr int kStageBuffers = 4;

// Barrier among the 128 epilogue threads only (barrier 0 belongs to __syncthreads).
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Barrier plus vote among the 128 epilogue threads: true when `mine` is true in all of them. The warps decide
// together whether to go on with a tile, so none of them can be left alone at the barrier above.
__device__ __forceinline__ bool epilogue_all(bool mine) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(mine))
      : "memory");
  return out != 0;
}

struct HalfEpilogue {
  __half* c;            // first element of this problem's C
  long long ldc;
  int m, n;
  float alpha, beta;
  bool use_tma;
  const CUtensorMap* map_c;
  uint8_t* staging;     // kStageBuffers * kStageBytes
  uint32_t load_bars;   // kStageBuffers mbarriers (shared-memory address of the first): "old C block has landed"
  int z;                // problem index (third map coordinate)
  bool hint_store;      // stores carry `store_policy` (results are written once and not read again by this launch)
  uint64_t store_policy;
};

// With beta != 0 the old values of a block are brought into the block's staging buffer by a TMA load (whole lines,
// asynchronous, issued two blocks ahead), combined in place and stored from the same buffer.
// Issued by the elected thread only. `block` is the running block count the load is for.
__device__ __forceinline__ void prefetch_old_block(const HalfEpilogue& e, int block, int cta_row0, int col) {
  const int b = block % kStageBuffers;
  const uint32_t bar = e.load_bars + 8u * b;
  mbar_arrive_expect_tx(bar, kStageBytes);
  tma_load_3d(smem_u32(e.staging + b * kStageBytes), e.map_c, bar, cta_row0, col, e.z);
}

// Start of a tile on the TMA path with beta != 0 (elected thread only): requests the old values of the tile's first
// two blocks. `stores` is the running block count; the two buffers involved were last read by the stores issued
// four and three blocks ago, both known to have finished.
__device__ __forceinline__ void prefetch_first_blocks(const HalfEpilogue& e, int stores, int cta_row0, int col0) {
  prefetch_old_block(e, stores, cta_row0, col0);
  if (col0 + kStageCols < e.n) prefetch_old_block(e, stores + 1, cta_row0, col0 + kStageCols);
}

// One 32-column block. `r` holds the fp32 accumulators of row `row` (global) = `row_in_cta` (0..127) of the CTA's
// 128 rows starting at `cta_row0`, columns [col, col + 32). `stores` counts the blocks this CTA has staged so far
// and `phases` holds one parity bit per load barrier (same values in all 128 threads); `elected` is true in exactly
// one thread. `use_beta`: old values take part (on the TMA path they were requested by prefetch_first_blocks or by
// an earlier call). `next_col` >= 0: the column at which the block two steps ahead of this one (same tile) starts.
// Returns false when the bounded wait for the old values expired.
__device__ __forceinline__ bool write_block(const HalfEpilogue& e, const uint32_t (&r)[32], int row, int row_in_cta,
                                            int cta_row0, int col, int next_col, bool use_beta, int& stores,
                                            uint32_t& phases, bool elected, unsigned int* status) {
  if (e.use_tma) {
    const int b = stores % kStageBuffers;
    uint8_t* const buf = e.staging + b * kStageBytes;
    __half* const mine = reinterpret_cast<__half*>(buf) + row_in_cta;
    if (use_beta) {
      if (!wait_old_block(e.load_bars + 8u * b, (phases >> b) & 1u, status)) return false;
      phases ^= 1u << b;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float v = e.alpha * __uint_as_float(r[j]);
      if (use_beta) v += e.beta * __half2float(mine[j * kStageRows]);
      mine[j * kStageRows] = __float2half_rn(v);
    }
    fence_proxy_async();  // the TMA unit reads the buffer through the async proxy
    epilogue_barrier();
    if (elected) {
      // a block that starts inside C is clipped by the TMA unit; one that lies wholly below C is not issued at all
      if (cta_row0 < e.m) {
        if (e.hint_store) tma_store_3d_hint(e.map_c, smem_u32(buf), cta_row0, col, e.z, e.store_policy);
        else tma_store_3d(e.map_c, smem_u32(buf), cta_row0, col, e.z);
      }
      bulk_commit();
      bulk_wait_read<2>();  // the store issued two blocks ago has left its buffer: block s + 2 lands there
      if (use_beta && next_col >= 0) prefetch_old_block(e, stores + 2, cta_row0, next_col);
    }
    ++stores;
    return true;
  }
  if (row < e.m) {
    __half* const cptr = e.c + static_cast<long long>(col) * e.ldc + row;
    float old[32];
    if (use_beta) {  // all loads before the first store: loads and stores through one pointer would serialise
#pragma unroll
      for (int j = 0; j < 32; ++j)
        old[j] = (col + j < e.n) ? __half2float(cptr[static_cast<long long>(j) * e.ldc]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col + j < e.n) {
        float v = e.alpha * __uint_as_float(r[j]);
        if (use_beta) v += e.beta * old[j];
        cptr[static_cast<long long>(j) * e.ldc] = __float2half_rn(v);
      }
    }
  }
  return true;
}

}  // namespace tc
}  // namespace b200
