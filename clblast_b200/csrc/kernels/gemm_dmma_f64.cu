// DGEMM on the FP64 tensor-core path (mma.sync m8n8k4 f64), for large double-precision GEMMs.
//
// tcgen05 has no FP64 mode, so double precision stays on warp-level instructions. The CUDA-core kernel
// (gemm_simt.cuh) issues one DFMA per 32 multiply-adds and tops out near two thirds of the FP64 pipe; one
// m8n8k4 DMMA performs 256 multiply-adds per warp instruction on the same pipe, which leaves issue slots for the
// shared-memory loads. Replaces, for large problems, the same reference code as the CUDA-core kernel (Xgemm /
// XgemmDirect: src/kernels/level3/xgemm_part3.opencl:53-305, xgemm_direct_part3.opencl:17-290). Tiles are staged
// exactly as in the CUDA-core kernel (any layout, leading dimension, offset and alignment; zero-filled edges).
// Each DMMA sums four k at a time, so results are not bit-identical to the k-ascending chain of the reference; the
// error against the exact product stays at the fp64 rounding level (asserted in the tests).
//
// CTA tile 128 x 128 x 16, 256 threads = 8 warps in a 4 (M) x 2 (N) grid, warp tile 32 x 64 = 4 x 8 DMMA blocks.
// Fragments (m8n8k4, A row-major, B column-major): lane = 4*g + t holds A(g, t), B(t, g), C(g, 2t) and C(g, 2t+1).
#include "gemm_simt.cuh"
#include "launchers.h"
#include "../runtime_state.h"

#include <cstdlib>
#include <cstring>

namespace b200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int NT = 256;
constexpr int LDS_A = BM + 4, LDS_B = BN + 4;  // row stride = 4 (mod 16) doubles: fragment loads are conflict-free
constexpr int SMEM_BYTES = 2 * BK * (LDS_A + LDS_B) * 8;  // double-buffered A and B tiles, above the 48 KB static limit

// CONV: op(A) is the implicit im2col matrix of image bz (rows = output pixels, contiguous along the pixels), gathered
// with the loader of the CUDA-core convolution (TileStager::fetch_conv); B holds the weights [filter][k].
template <bool A_KC, bool B_KC, bool CONV = false>
__global__ void __launch_bounds__(NT, 1) gemm_dmma_kernel(const SimtParams<double> p) {
  using Tr = TraitsF64;
  using StA = TileStager<Tr, BM, BK, NT, A_KC>;
  using StB = TileStager<Tr, BN, BK, NT, B_KC>;
  extern __shared__ __align__(16) unsigned char dmma_smem[];
  double(*sA)[BK * LDS_A] = reinterpret_cast<double(*)[BK * LDS_A]>(dmma_smem);
  double(*sB)[BK * LDS_B] = reinterpret_cast<double(*)[BK * LDS_B]>(dmma_smem + sizeof(double) * 2 * BK * LDS_A);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm = (warp & 3) * 32;   // warp tile origin inside the CTA tile
  const int wn = (warp >> 2) * 64;
  const bool a_vec_ok = (p.lda % 2) == 0, b_vec_ok = (p.ldb % 2) == 0;

  for (long long tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
    // Tiles are walked in groups of eight tile rows by all tile columns (rows fastest inside a group), so the CTAs
    // running at the same time share a few operand rows and columns in L2 instead of sweeping all of A.
    const long long per_problem = p.tiles_m * p.tiles_n;
    const long long bz = tile / per_problem;
    const long long in_problem = tile - bz * per_problem;
    const long long per_group = 8 * p.tiles_n;
    const long long group = in_problem / per_group;
    const long long first_m = group * 8;
    const long long rows = (p.tiles_m - first_m) < 8 ? (p.tiles_m - first_m) : 8;
    const long long in_group = in_problem - group * per_group;
    const long long tm = first_m + in_group % rows;
    const long long tn = in_group / rows;
    const long long m0 = tm * BM, n0 = tn * BN;
    const long long m_rem = p.m - m0, n_rem = p.n - n0;
    // rank-k updates: tiles wholly outside the triangle are not computed (the branch is uniform over the CTA)
    if ((p.tri == 1 && m0 > n0 + BN - 1) || (p.tri == 2 && n0 > m0 + BM - 1)) continue;
    const double* a_base = static_cast<const double*>(p.a) + (p.a_offs ? p.a_offs[bz] : p.a_off + bz * p.a_stride);
    const double* b_base = static_cast<const double*>(p.b) + (p.b_offs ? p.b_offs[bz] : p.b_off + bz * p.b_stride);
    double* c_base = static_cast<double*>(p.c) + (p.c_offs ? p.c_offs[bz] : p.c_off + bz * p.c_stride);
    const double alpha = p.alphas ? p.alphas[bz] : p.alpha;
    const double beta = p.betas ? p.betas[bz] : p.beta;

    double acc[4][8][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    double ra[StA::NV][Tr::VEC], rb[StB::NV][Tr::VEC];
    int conv_h0[CONV ? StA::NV : 1][CONV ? Tr::VEC : 1];
    int conv_w0[CONV ? StA::NV : 1][CONV ? Tr::VEC : 1];
    if constexpr (CONV) StA::conv_pixels(conv_h0, conv_w0, p.conv, m0, m_rem, tid);
    auto fetch_tiles = [&](long long k0) {
      if constexpr (CONV) {
        StA::fetch_conv(ra, a_base, p.conv, conv_h0, conv_w0, k0, p.k - k0, tid);
      } else {
        StA::fetch(ra, a_base, p.lda, m0, k0, m_rem, p.k - k0, a_vec_ok, tid);
      }
      StB::fetch(rb, b_base, p.ldb, n0, k0, n_rem, p.k - k0, b_vec_ok, tid);
    };
    fetch_tiles(0);
    __syncthreads();
    StA::template stash<LDS_A>(sA[0], ra, false, tid);
    StB::template stash<LDS_B>(sB[0], rb, false, tid);
    __syncthreads();

    int cur = 0;
    for (long long k0 = 0; k0 < p.k; k0 += BK) {
      const bool has_next = (k0 + BK) < p.k;
      if (has_next) fetch_tiles(k0 + BK);
      const double* __restrict__ As = sA[cur];
      const double* __restrict__ Bs = sB[cur];
#pragma unroll
      for (int ks = 0; ks < BK; ks += 4) {
        double af[4], bf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) af[i] = As[(ks + t) * LDS_A + wm + i * 8 + g];
#pragma unroll
        for (int j = 0; j < 8; ++j) bf[j] = Bs[(ks + t) * LDS_B + wn + j * 8 + g];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(acc[i][j][0]), "+d"(acc[i][j][1])
                         : "d"(af[i]), "d"(bf[j]));
        // The next K block goes to the other buffer half-way through this one: nobody reads that buffer any more
        // (everyone passed the barrier below after its last use), and the stores, bank conflicts of the transposing
        // ones included, run under the remaining DMMAs instead of leaving the FP64 pipe idle.
        if (ks == BK / 2 - 4 && has_next) {
          StA::template stash<LDS_A>(sA[cur ^ 1], ra, false, tid);
          StB::template stash<LDS_B>(sB[cur ^ 1], rb, false, tid);
        }
      }
      if (has_next) {
        __syncthreads();
        cur ^= 1;
      }
    }

    // Epilogue: alpha*acc (+ beta*c; C is only read when beta != 0), same fused form as the CUDA-core kernel.
    const bool use_beta = beta != 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const long long nn = wn + j * 8 + 2 * t + h;
        if (nn >= n_rem) continue;
        double* c_col = c_base + (n0 + nn) * p.ldc + m0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const long long mm = wm + i * 8 + g;
          if (mm < m_rem && (p.tri == 0 || (p.tri == 1 ? m0 + mm <= n0 + nn : m0 + mm >= n0 + nn))) {
            const double r = acc[i][j][h];
            c_col[mm] = use_beta ? fma(beta, c_col[mm], __dmul_rn(alpha, r)) : __dmul_rn(alpha, r);
          }
        }
      }
    }
  }
}

template <bool A_KC, bool B_KC, bool CONV = false>
cudaError_t go(const GemmDesc& d, cudaStream_t stream) {
  SimtParams<double> p;
  p.a = d.a; p.b = d.b; p.c = d.c;
  p.m = d.m; p.n = d.n; p.k = d.k;
  p.lda = d.lda; p.ldb = d.ldb; p.ldc = d.ldc;
  p.a_off = d.a_off; p.b_off = d.b_off; p.c_off = d.c_off;
  p.a_stride = d.a_stride; p.b_stride = d.b_stride; p.c_stride = d.c_stride;
  p.a_offs = d.a_offs; p.b_offs = d.b_offs; p.c_offs = d.c_offs;
  p.alphas = static_cast<const double*>(d.alphas);
  p.betas = static_cast<const double*>(d.betas);
  p.alpha = d.alpha[0];
  p.beta = d.beta[0];
  p.batch = d.batch;
  p.tiles_m = (d.m + BM - 1) / BM;
  p.tiles_n = (d.n + BN - 1) / BN;
  p.total_tiles = p.tiles_m * p.tiles_n * d.batch;
  p.conj_a = p.conj_b = 0;
  p.tri = d.tri;
  p.real_diag = 0;
  p.conv = d.conv;
  const long long max_grid = 1LL << 30;
  const unsigned grid = static_cast<unsigned>(p.total_tiles < max_grid ? p.total_tiles : max_grid);
  const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(gemm_dmma_kernel<A_KC, B_KC, CONV>), SMEM_BYTES);
  if (e != cudaSuccess) return e;
  gemm_dmma_kernel<A_KC, B_KC, CONV><<<grid, NT, SMEM_BYTES, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_dmma_f64(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 64 || d.is_conv || d.force_small) return cudaErrorNotSupported;
  static const bool forced_dfma = [] {
    const char* v = std::getenv("B200BLAS_DGEMM");
    return v != nullptr && std::strcmp(v, "dfma") == 0;
  }();
  if (forced_dfma) return cudaErrorNotSupported;
  // enough 128x128 tiles to fill the machine; smaller problems keep the k-ascending CUDA-core kernel
  const long long tiles = ((d.m + BM - 1) / BM) * ((d.n + BN - 1) / BN) * d.batch;
  if (d.m < 96 || d.n < 96 || d.k < 32 || tiles < 120) return cudaErrorNotSupported;
  *name = "dmma_f64_128x128x16";
  if (d.a_kcontig) return d.b_kcontig ? go<true, true>(d, stream) : go<true, false>(d, stream);
  return d.b_kcontig ? go<false, true>(d, stream) : go<false, false>(d, stream);
}

// Double-precision Convgemm as an implicit GEMM on the FP64 tensor-core path: no column matrix in memory. Replaces the
// reference's XconvgemmNormal / XconvgemmFlip for large problems (src/kernels/levelx/xconvgemm_part2.opencl:27-336).
cudaError_t launch_dmma_conv_f64(const GemmDesc& d, cudaStream_t stream, const char** name) {
  if (d.dtype != 64 || !d.is_conv || d.force_small) return cudaErrorNotSupported;
  static const bool disabled = [] {  // B200BLAS_CONV=simt | im2col: the CUDA-core kernel / the two-step route
    const char* v = std::getenv("B200BLAS_CONV");
    return v != nullptr && (std::strcmp(v, "simt") == 0 || std::strcmp(v, "im2col") == 0);
  }();
  if (disabled) return cudaErrorNotSupported;
  const long long tiles = ((d.m + BM - 1) / BM) * ((d.n + BN - 1) / BN) * d.batch;
  if (d.m < 96 || d.n < 32 || d.k < 32 || tiles < 120) return cudaErrorNotSupported;
  if (d.m > 0x7FFFFFFF || d.k > 0x7FFFFFFF) return cudaErrorNotSupported;  // the loader keeps pixels and K rows in int
  *name = "conv_dmma_f64_128x128x16";
  return go<false, true, true>(d, stream);
}

}  // namespace b200
