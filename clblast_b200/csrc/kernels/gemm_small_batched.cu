// Streaming kernel for large batches of small fp32 GEMMs (each whole problem fits one tile).
//
// Replaces XgemmDirectBatched* / XgemmDirectStridedBatched* of the reference
// (src/kernels/level3/xgemm_direct_batched.opencl:24-212, launched from
// src/routines/levelx/xgemmstridedbatched.cpp:215-257 and xgemmbatched.cpp:229-295) for the shapes where those
// routines are bound by memory traffic, not arithmetic: thousands of 32x32x32-class or 64x128x96-class products.
// Each CTA is persistent and walks over its share of the batch; the operands (and C when beta != 0) of the NEXT
// problem are copied global -> shared with cp.async while the current one is multiplied out of shared memory, so
// there are always tens of KB of loads in flight per SM and no register staging.
//
// Arithmetic order per output element is the reference's (acc = 0; k ascending fused multiply-add; then
// alpha*acc or fma(beta, c, alpha*acc)), so results are bit-identical to the generic CUDA-core kernel.
//
// Requirements (checked on the host, otherwise the generic kernel runs): fp32, m <= BM, n <= BN, k <= KMAX, every
// contiguous extent a multiple of 4 elements, 16-byte aligned bases, leading dimensions, strides and offsets.
#include <cuda_runtime.h>
#include <stdint.h>

#include "launchers.h"
#include "../runtime_state.h"

namespace b200 {

namespace {

struct SmallParams {
  const float* a;
  const float* b;
  float* c;
  int m, n, k;
  long long lda, ldb, ldc;
  long long a_off, b_off, c_off, a_stride, b_stride, c_stride;
  const long long* a_offs;
  const long long* b_offs;
  const long long* c_offs;
  const float* alphas;
  const float* betas;
  float alpha, beta;
  long long batch;
  int need_c;  // some beta is non-zero: C tiles are prefetched too
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shared-memory footprint of one operand buffer set (A, B, C) of one group, in floats.
template <int BM, int BN, int KMAX, bool A_KC, bool B_KC>
struct SmallLayout {
  static constexpr int LDA = A_KC ? KMAX + 4 : BM + 4;  // row stride of the A tile
  static constexpr int LDB = B_KC ? KMAX + 4 : BN + 4;
  static constexpr int A_FLOATS = (A_KC ? BM : KMAX) * LDA;
  static constexpr int B_FLOATS = (B_KC ? BN : KMAX) * LDB;
  static constexpr int C_FLOATS = BM * BN;  // [n][BM]
  static constexpr int SET_FLOATS = A_FLOATS + B_FLOATS + C_FLOATS;
};

// SETS = 2: the next problem is prefetched while the current one is computed (double buffering inside the CTA).
// SETS = 1: one buffer set per CTA; two CTAs share an SM and overlap each other's loads and arithmetic.
// CTAS: resident CTAs per SM the launch is sized for (and the register bound that goes with it).
template <int BM, int BN, int KMAX, int TM, int TN, int GROUPS, int SETS, int CTAS, bool A_KC, bool B_KC>
__global__ void __launch_bounds__((BM / TM) * (BN / TN) * GROUPS, CTAS) gemm_small_batched_kernel(const SmallParams p) {
  using L = SmallLayout<BM, BN, KMAX, A_KC, B_KC>;
  constexpr int NT = (BM / TM) * (BN / TN);
  extern __shared__ __align__(16) float smem[];

  const int group = threadIdx.x / NT;
  const int tid = threadIdx.x % NT;
  const int tx = tid % (BM / TM);
  const int ty = tid / (BM / TM);
  float* const my_sets = smem + static_cast<size_t>(group) * SETS * L::SET_FLOATS;

  // Zero everything once: positions outside (m, n, k) are never written again and multiply as zeros.
  for (int i = threadIdx.x; i < GROUPS * SETS * L::SET_FLOATS; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();

  const long long stride_tiles = static_cast<long long>(gridDim.x) * GROUPS;
  const long long first = static_cast<long long>(blockIdx.x) * GROUPS + group;
  const long long rounds = (p.batch - static_cast<long long>(blockIdx.x) * GROUPS + stride_tiles - 1) / stride_tiles;

  auto bases = [&](long long t, const float*& a, const float*& b, float*& c) {
    a = p.a + (p.a_offs ? p.a_offs[t] : p.a_off + t * p.a_stride);
    b = p.b + (p.b_offs ? p.b_offs[t] : p.b_off + t * p.b_stride);
    c = p.c + (p.c_offs ? p.c_offs[t] : p.c_off + t * p.c_stride);
  };

  // Copy plan of one operand: `rows` runs of `run` 16-byte chunks. Each thread walks the chunk list with stride NT;
  // the (row, chunk) pair is advanced incrementally so the loop contains no integer division.
  struct Plan {
    int run, rows, row0, ch0, drow, dch;
  };
  auto make_plan = [&](int run, int rows) {
    Plan q;
    q.run = run; q.rows = rows;
    q.row0 = tid / run; q.ch0 = tid % run;
    q.drow = NT / run; q.dch = NT % run;
    return q;
  };
  const Plan plan_a = make_plan((A_KC ? p.k : p.m) / 4, A_KC ? p.m : p.k);
  const Plan plan_b = make_plan((B_KC ? p.k : p.n) / 4, B_KC ? p.n : p.k);
  const Plan plan_c = make_plan(p.m / 4, p.n);

  auto copy_operand = [&](const Plan& q, float* dst, int dst_ld, const float* src, long long src_ld) {
    int r = q.row0, ch = q.ch0;
    while (r < q.rows) {
      cp_async16(dst + r * dst_ld + ch * 4, src + static_cast<long long>(r) * src_ld + ch * 4);
      r += q.drow;
      ch += q.dch;
      if (ch >= q.run) { ch -= q.run; ++r; }
    }
  };

  auto prefetch = [&](long long t, int set) {
    if (t >= p.batch) return;
    const float *a, *b;
    float* c;
    bases(t, a, b, c);
    float* sa = my_sets + set * L::SET_FLOATS;
    float* sb = sa + L::A_FLOATS;
    float* sc = sb + L::B_FLOATS;
    copy_operand(plan_a, sa, L::LDA, a, p.lda);
    copy_operand(plan_b, sb, L::LDB, b, p.ldb);
    if (p.need_c) copy_operand(plan_c, sc, BM, c, p.ldc);
  };

  if (SETS == 2) {
    prefetch(first, 0);
    cp_async_commit();
  }

  for (long long round = 0; round < rounds; ++round) {
    const long long t = first + round * stride_tiles;
    const int set = (SETS == 2) ? static_cast<int>(round & 1) : 0;
    if (SETS == 2) {
      prefetch(t + stride_tiles, set ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      prefetch(t, 0);
      cp_async_commit();
      cp_async_wait<0>();
    }
    __syncthreads();

    if (t < p.batch) {
      const float* sa = my_sets + set * L::SET_FLOATS;
      const float* sb = sa + L::A_FLOATS;
      const float* sc = sb + L::B_FLOATS;
      float acc[TM][TN];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

      // Four k per step: operands whose K is contiguous in shared memory are read as one float4 per row, which is
      // free of bank conflicts; the multiply-adds still run in ascending k for every output element.
      const int k4 = p.k & ~3;
      for (int kk = 0; kk < k4; kk += 4) {
        float av[4][TM], bv[4][TN];
#pragma unroll
        for (int cm = 0; cm < TM / 4; ++cm) {
          const int m0 = cm * (BM / (TM / 4)) + tx * 4;
          if (A_KC) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 v = *reinterpret_cast<const float4*>(sa + (m0 + i) * L::LDA + kk);
              av[0][cm * 4 + i] = v.x; av[1][cm * 4 + i] = v.y; av[2][cm * 4 + i] = v.z; av[3][cm * 4 + i] = v.w;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 v = *reinterpret_cast<const float4*>(sa + (kk + q) * L::LDA + m0);
              av[q][cm * 4 + 0] = v.x; av[q][cm * 4 + 1] = v.y; av[q][cm * 4 + 2] = v.z; av[q][cm * 4 + 3] = v.w;
            }
          }
        }
#pragma unroll
        for (int cn = 0; cn < TN / 4; ++cn) {
          const int n0 = cn * (BN / (TN / 4)) + ty * 4;
          if (B_KC) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float4 v = *reinterpret_cast<const float4*>(sb + (n0 + j) * L::LDB + kk);
              bv[0][cn * 4 + j] = v.x; bv[1][cn * 4 + j] = v.y; bv[2][cn * 4 + j] = v.z; bv[3][cn * 4 + j] = v.w;
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 v = *reinterpret_cast<const float4*>(sb + (kk + q) * L::LDB + n0);
              bv[q][cn * 4 + 0] = v.x; bv[q][cn * 4 + 1] = v.y; bv[q][cn * 4 + 2] = v.z; bv[q][cn * 4 + 3] = v.w;
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
          for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[q][i], bv[q][j], acc[i][j]);
      }
      for (int kk = k4; kk < p.k; ++kk) {  // k tail (only when neither operand is K-contiguous)
        float av[TM], bv[TN];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
          const int mi = (i / 4) * (BM / (TM / 4)) + tx * 4 + (i & 3);
          av[i] = A_KC ? sa[mi * L::LDA + kk] : sa[kk * L::LDA + mi];
        }
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          const int nj = (j / 4) * (BN / (TN / 4)) + ty * 4 + (j & 3);
          bv[j] = B_KC ? sb[nj * L::LDB + kk] : sb[kk * L::LDB + nj];
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }

      const float *ga, *gb;
      float* gc;
      bases(t, ga, gb, gc);
      const float alpha = p.alphas ? p.alphas[t] : p.alpha;
      const float beta = p.betas ? p.betas[t] : p.beta;
      const bool use_beta = beta != 0.f;
#pragma unroll
      for (int cn = 0; cn < TN / 4; ++cn) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int nn = cn * (BN / (TN / 4)) + ty * 4 + j;
          if (nn >= p.n) continue;
#pragma unroll
          for (int cm = 0; cm < TM / 4; ++cm) {
            const int mm = cm * (BM / (TM / 4)) + tx * 4;
            if (mm >= p.m) continue;  // m is a multiple of 4, so a chunk is either whole or absent
            float4 out;
            const float r0 = acc[cm * 4 + 0][cn * 4 + j], r1 = acc[cm * 4 + 1][cn * 4 + j];
            const float r2 = acc[cm * 4 + 2][cn * 4 + j], r3 = acc[cm * 4 + 3][cn * 4 + j];
            if (use_beta) {
              const float4 old = *reinterpret_cast<const float4*>(sc + nn * BM + mm);
              out.x = fmaf(beta, old.x, __fmul_rn(alpha, r0));
              out.y = fmaf(beta, old.y, __fmul_rn(alpha, r1));
              out.z = fmaf(beta, old.z, __fmul_rn(alpha, r2));
              out.w = fmaf(beta, old.w, __fmul_rn(alpha, r3));
            } else {
              out.x = __fmul_rn(alpha, r0);
              out.y = __fmul_rn(alpha, r1);
              out.z = __fmul_rn(alpha, r2);
              out.w = __fmul_rn(alpha, r3);
            }
            *reinterpret_cast<float4*>(gc + static_cast<long long>(nn) * p.ldc + mm) = out;
          }
        }
      }
    }
    __syncthreads();  // the set just read is the target of the next prefetch
  }
  cp_async_wait<0>();
}

template <int BM, int BN, int KMAX, int TM, int TN, int GROUPS, int SETS, int CTAS = 2>
struct SmallLauncher {
  template <bool A_KC, bool B_KC>
  static cudaError_t go(const SmallParams& p, cudaStream_t stream, int sm_count) {
    using L = SmallLayout<BM, BN, KMAX, A_KC, B_KC>;
    constexpr int SMEM = GROUPS * SETS * L::SET_FLOATS * static_cast<int>(sizeof(float));
    static_assert(CTAS * SMEM <= 226 * 1024, "the resident CTAs must fit the shared memory of one SM");
    auto kernel = gemm_small_batched_kernel<BM, BN, KMAX, TM, TN, GROUPS, SETS, CTAS, A_KC, B_KC>;
    {  // per-context attribute (remembered per context)
      const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), SMEM);
      if (e != cudaSuccess) return e;
    }
    const long long ctas = (p.batch + GROUPS - 1) / GROUPS;
    const long long resident = static_cast<long long>(CTAS) * sm_count;
    const int grid = static_cast<int>(ctas < resident ? ctas : resident);
    constexpr int NT = (BM / TM) * (BN / TN) * GROUPS;
    kernel<<<grid, NT, SMEM, stream>>>(p);
    return cudaGetLastError();
  }

  static cudaError_t launch(const SmallParams& p, bool a_kc, bool b_kc, cudaStream_t stream, int sm_count) {
    if (a_kc) return b_kc ? go<true, true>(p, stream, sm_count) : go<true, false>(p, stream, sm_count);
    return b_kc ? go<false, true>(p, stream, sm_count) : go<false, false>(p, stream, sm_count);
  }
};

bool aligned4(long long v) { return (v & 3) == 0; }

}  // namespace

cudaError_t launch_small_batched_f32(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 32 || d.is_conv || d.force_small || d.conj_a || d.conj_b || d.tri) return cudaErrorNotSupported;
  if (d.batch < 296) return cudaErrorNotSupported;  // fewer than two problems per SM: the generic kernel is fine
  const bool fits_small = d.m <= 32 && d.n <= 32 && d.k <= 32;
  const bool fits_wide = d.m <= 64 && d.n <= 128 && d.k <= 96;
  if (!fits_small && !fits_wide) return cudaErrorNotSupported;
  // 16-byte granularity everywhere: extents along contiguous dimensions, leading dimensions, offsets, strides
  const long long a_run = d.a_kcontig ? d.k : d.m, b_run = d.b_kcontig ? d.k : d.n;
  if (!aligned4(a_run) || !aligned4(b_run) || !aligned4(d.m)) return cudaErrorNotSupported;
  if (!aligned4(d.lda) || !aligned4(d.ldb) || !aligned4(d.ldc)) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(d.a) | reinterpret_cast<uintptr_t>(d.b) | reinterpret_cast<uintptr_t>(d.c)) & 15)
    return cudaErrorNotSupported;
  if (d.a_offs) {
    // per-batch offsets live on the device; the staged tables are only eligible when the host marked them aligned
    if (!d.tables_aligned4) return cudaErrorNotSupported;
  } else if (!aligned4(d.a_off) || !aligned4(d.b_off) || !aligned4(d.c_off) || !aligned4(d.a_stride) ||
             !aligned4(d.b_stride) || !aligned4(d.c_stride)) {
    return cudaErrorNotSupported;
  }

  SmallParams p;
  p.a = static_cast<const float*>(d.a);
  p.b = static_cast<const float*>(d.b);
  p.c = static_cast<float*>(d.c);
  p.m = static_cast<int>(d.m); p.n = static_cast<int>(d.n); p.k = static_cast<int>(d.k);
  p.lda = d.lda; p.ldb = d.ldb; p.ldc = d.ldc;
  p.a_off = d.a_off; p.b_off = d.b_off; p.c_off = d.c_off;
  p.a_stride = d.a_stride; p.b_stride = d.b_stride; p.c_stride = d.c_stride;
  p.a_offs = d.a_offs; p.b_offs = d.b_offs; p.c_offs = d.c_offs;
  p.alphas = static_cast<const float*>(d.alphas);
  p.betas = static_cast<const float*>(d.betas);
  p.alpha = static_cast<float>(d.alpha[0]);
  p.beta = static_cast<float>(d.beta[0]);
  p.batch = d.batch;
  p.need_c = (d.betas != nullptr) || (p.beta != 0.f);

  const int device_sms = sm_count();
  if (device_sms <= 0) return cudaErrorNotSupported;

  // Thread tiles of 4 x 4 (8 x 4 for the wide class) keep several warps per scheduler busy: with 8 x 8 tiles a
  // scheduler had a single warp and issued at 0.42 instructions per cycle.
  if (fits_small) {
    *name = "small_batched_f32_32x32x32";
    return SmallLauncher<32, 32, 32, 4, 4, 1, 2, 8>::launch(p, d.a_kcontig, d.b_kcontig, stream, device_sms);
  }
  *name = "small_batched_f32_64x128x96";
  return SmallLauncher<64, 128, 96, 8, 4, 1, 1>::launch(p, d.a_kcontig, d.b_kcontig, stream, device_sms);
}

}  // namespace b200
