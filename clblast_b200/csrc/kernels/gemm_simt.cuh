// Register-tiled CUDA-core GEMM for any dtype, transpose, leading dimension, offset and alignment.
//
// This is the B200 replacement for the reference's whole "direct" family (XgemmDirect{NN,NT,TN,TT},
// XgemmDirectBatched*, XgemmDirectStridedBatched*, XconvgemmNormal/Flip:
// src/kernels/level3/xgemm_direct_part3.opencl:17-290, xgemm_direct_batched.opencl:24-212,
// src/kernels/levelx/xconvgemm_part2.opencl:27-336) and, for fp32/fp64/complex, also for the "indirect"
// Xgemm kernel together with its copy/pad/transpose pre- and post-kernels
// (src/kernels/level3/xgemm_part3.opencl:53-305, copy_pad.opencl, transpose_pad.opencl): edge tiles and
// transposed operands are handled while staging tiles into shared memory, so no padded temporaries exist.
//
// Arithmetic order per output element follows the reference: acc = 0; for k ascending: acc += a*b (fused),
// then alpha*acc (+ beta*c only when beta != 0, so C is write-only for beta == 0)
// (xgemm_direct_part3.opencl:41-135, src/kernels/common.opencl:208-244). Half inputs are accumulated in fp32.
//
// The problem is normalised by the host to a column-major C (M contiguous); op(A) is M x K and is either
// M-contiguous (element (i,l) at l*lda+i) or K-contiguous (i*lda+l); op(B) is K x N and is either
// K-contiguous (j*ldb+l) or N-contiguous (l*ldb+j).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_desc.h"
#include "../runtime_state.h"

namespace b200 {

template <typename S>
struct SimtParams {
  const void* a;
  const void* b;
  void* c;
  long long m, n, k, lda, ldb, ldc;
  long long a_off, b_off, c_off, a_stride, b_stride, c_stride;
  const long long* a_offs;
  const long long* b_offs;
  const long long* c_offs;
  const S* alphas;
  const S* betas;
  S alpha, beta;
  long long batch;
  long long tiles_m, tiles_n, total_tiles;
  int conj_a, conj_b;
  int tri, real_diag;  // triangle mask and real diagonal of the rank-k updates (see GemmDesc)
  ConvGeom conv;
};

// ---- per-dtype arithmetic -----------------------------------------------------------------------------

struct TraitsF32 {
  using T = float;
  using S = float;
  static constexpr int VEC = 4;  // elements per 16-byte global access
  static constexpr int CW = 4;   // compute-type elements per 16-byte shared access
  static __device__ __forceinline__ S ld(T v) { return v; }
  static __device__ __forceinline__ T st(S v) { return v; }
  static __device__ __forceinline__ S zero() { return 0.f; }
  static __device__ __forceinline__ S conj(S v) { return v; }
  static __device__ __forceinline__ S real_only(S v) { return v; }
  static __device__ __forceinline__ void mad(S& c, S a, S b) { c = fmaf(a, b, c); }
  static __device__ __forceinline__ S mul(S a, S b) { return __fmul_rn(a, b); }
  // alpha*x + beta*y as fma(beta, y, alpha*x): the fused form of the reference's AXPBY, bit-identical to the
  // reference kernels compiled with contraction (and to the CPU oracle).
  static __device__ __forceinline__ S axpby(S al, S x, S be, S y) { return fmaf(be, y, __fmul_rn(al, x)); }
  static __device__ __forceinline__ bool is_zero(S v) { return v == 0.f; }
  static __host__ S from_host(const double* v) { return static_cast<float>(v[0]); }
};

struct TraitsF64 {
  using T = double;
  using S = double;
  static constexpr int VEC = 2;
  static constexpr int CW = 2;
  static __device__ __forceinline__ S ld(T v) { return v; }
  static __device__ __forceinline__ T st(S v) { return v; }
  static __device__ __forceinline__ S zero() { return 0.0; }
  static __device__ __forceinline__ S conj(S v) { return v; }
  static __device__ __forceinline__ S real_only(S v) { return v; }
  static __device__ __forceinline__ void mad(S& c, S a, S b) { c = fma(a, b, c); }
  static __device__ __forceinline__ S mul(S a, S b) { return __dmul_rn(a, b); }
  static __device__ __forceinline__ S axpby(S al, S x, S be, S y) { return fma(be, y, __dmul_rn(al, x)); }
  static __device__ __forceinline__ bool is_zero(S v) { return v == 0.0; }
  static __host__ S from_host(const double* v) { return v[0]; }
};

struct TraitsF16 {
  using T = __half;
  using S = float;
  static constexpr int VEC = 8;
  static constexpr int CW = 4;
  static __device__ __forceinline__ S ld(T v) { return __half2float(v); }
  static __device__ __forceinline__ T st(S v) { return __float2half_rn(v); }
  static __device__ __forceinline__ S zero() { return 0.f; }
  static __device__ __forceinline__ S conj(S v) { return v; }
  static __device__ __forceinline__ S real_only(S v) { return v; }
  static __device__ __forceinline__ void mad(S& c, S a, S b) { c = fmaf(a, b, c); }
  static __device__ __forceinline__ S mul(S a, S b) { return a * b; }
  static __device__ __forceinline__ S axpby(S al, S x, S be, S y) { return al * x + be * y; }
  static __device__ __forceinline__ bool is_zero(S v) { return v == 0.f; }
  static __host__ S from_host(const double* v) { return static_cast<float>(v[0]); }
};

struct TraitsC32 {
  using T = float2;
  using S = float2;
  static constexpr int VEC = 2;
  static constexpr int CW = 2;
  static __device__ __forceinline__ S ld(T v) { return v; }
  static __device__ __forceinline__ T st(S v) { return v; }
  static __device__ __forceinline__ S zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ S conj(S v) { return make_float2(v.x, -v.y); }
  static __device__ __forceinline__ S real_only(S v) { return make_float2(v.x, 0.f); }
  static __device__ __forceinline__ void mad(S& c, S a, S b) {
    c.x = fmaf(a.x, b.x, c.x);
    c.x = fmaf(-a.y, b.y, c.x);
    c.y = fmaf(a.x, b.y, c.y);
    c.y = fmaf(a.y, b.x, c.y);
  }
  static __device__ __forceinline__ S mul(S a, S b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
  static __device__ __forceinline__ S axpby(S al, S x, S be, S y) {
    S p = mul(al, x), q = mul(be, y);
    return make_float2(p.x + q.x, p.y + q.y);
  }
  static __device__ __forceinline__ bool is_zero(S v) { return v.x == 0.f && v.y == 0.f; }
  static __host__ S from_host(const double* v) { return make_float2(static_cast<float>(v[0]), static_cast<float>(v[1])); }
};

struct TraitsC64 {
  using T = double2;
  using S = double2;
  static constexpr int VEC = 1;
  static constexpr int CW = 1;
  static __device__ __forceinline__ S ld(T v) { return v; }
  static __device__ __forceinline__ T st(S v) { return v; }
  static __device__ __forceinline__ S zero() { return make_double2(0.0, 0.0); }
  static __device__ __forceinline__ S conj(S v) { return make_double2(v.x, -v.y); }
  static __device__ __forceinline__ S real_only(S v) { return make_double2(v.x, 0.0); }
  static __device__ __forceinline__ void mad(S& c, S a, S b) {
    c.x = fma(a.x, b.x, c.x);
    c.x = fma(-a.y, b.y, c.x);
    c.y = fma(a.x, b.y, c.y);
    c.y = fma(a.y, b.x, c.y);
  }
  static __device__ __forceinline__ S mul(S a, S b) { return make_double2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }
  static __device__ __forceinline__ S axpby(S al, S x, S be, S y) {
    S p = mul(al, x), q = mul(be, y);
    return make_double2(p.x + q.x, p.y + q.y);
  }
  static __device__ __forceinline__ bool is_zero(S v) { return v.x == 0.0 && v.y == 0.0; }
  static __host__ S from_host(const double* v) { return make_double2(v[0], v[1]); }
};

template <typename T, int N>
struct alignas(sizeof(T) * N) VecOf {
  T v[N];
};

// ---- tile staging ---------------------------------------------------------------------------------------

// One operand tile is BX (the M or N extent) by BK. Every thread owns NV vectors of VEC elements taken along the
// operand's contiguous dimension. `fetch` brings them into registers (16-byte loads when the tile is interior
// and 16-byte aligned, predicated scalar loads with zero fill otherwise); `stash` writes them to the
// shared tile, which is always laid out [BK][BX + PAD] in the compute type.
template <typename Tr, int BX, int BK, int NT, bool KCONTIG>
struct TileStager {
  using T = typename Tr::T;
  using S = typename Tr::S;
  static constexpr int VEC = Tr::VEC;
  static constexpr int NVEC = BX * BK / VEC;
  static constexpr int NV = NVEC / NT;
  static_assert(NVEC % NT == 0 && NV >= 1, "tile does not divide over the threads");
  static constexpr int VPR = (KCONTIG ? BK : BX) / VEC;  // vectors per contiguous run
  static_assert((KCONTIG ? BK : BX) % VEC == 0, "contiguous extent must be a whole number of vectors");

  static __device__ __forceinline__ void coords(int i, int tid, int& x, int& kk) {
    const int v = tid + i * NT;
    if (KCONTIG) {
      kk = (v % VPR) * VEC;
      x = v / VPR;
    } else {
      x = (v % VPR) * VEC;
      kk = v / VPR;
    }
  }

  // base points at element (x0, k0 = 0) of the operand for this batch; x_rem / k_rem are the extents left
  // from the tile origin (may exceed the tile size).
  static __device__ __forceinline__ void fetch(T (&reg)[NV][VEC], const T* __restrict__ base, long long ld,
                                               long long x0, long long k0, long long x_rem, long long k_rem,
                                               bool ld_vec_ok, int tid) {
    const T* tile = KCONTIG ? base + x0 * ld + k0 : base + k0 * ld + x0;
    const bool fast = ld_vec_ok && x_rem >= BX && k_rem >= BK && ((reinterpret_cast<uintptr_t>(tile) & 15) == 0);
    if (fast) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        int x, kk;
        coords(i, tid, x, kk);
        const T* src = KCONTIG ? tile + static_cast<long long>(x) * ld + kk : tile + static_cast<long long>(kk) * ld + x;
        const VecOf<T, VEC> vv = *reinterpret_cast<const VecOf<T, VEC>*>(src);
#pragma unroll
        for (int j = 0; j < VEC; ++j) reg[i][j] = vv.v[j];
      }
    } else {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        int x, kk;
        coords(i, tid, x, kk);
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
          const int xe = KCONTIG ? x : x + j;
          const int ke = KCONTIG ? kk + j : kk;
          T val;
          if (xe < x_rem && ke < k_rem) {
            val = KCONTIG ? tile[static_cast<long long>(xe) * ld + ke] : tile[static_cast<long long>(ke) * ld + xe];
          } else {
            val = Tr::st(Tr::zero());
          }
          reg[i][j] = val;
        }
      }
    }
  }

  // Convolution flavour of `fetch` for op(A): x indexes output pixels, k indexes (channel, kh, kw). The pixel part of
  // the address (top-left tap of every output pixel this thread stages) does not change along K, so it is computed
  // once per tile by conv_pixels(); pixels outside the tile get a row far outside the image and load as zero.
  static __device__ __forceinline__ void conv_pixels(int (&hi0)[NV][VEC], int (&wi0)[NV][VEC], const ConvGeom& g,
                                                     long long x0, long long x_rem, int tid) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      int x, kk;
      coords(i, tid, x, kk);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const int xe = x + j;
        if (xe < x_rem) {
          const int p = static_cast<int>(x0) + xe;
          const int ho = p / g.out_w;
          const int wo = p - ho * g.out_w;
          hi0[i][j] = ho * g.stride_h - g.pad_h;
          wi0[i][j] = wo * g.stride_w - g.pad_w;
        } else {
          hi0[i][j] = -(1 << 28);
          wi0[i][j] = 0;
        }
      }
    }
  }

  static __device__ __forceinline__ void fetch_conv(T (&reg)[NV][VEC], const T* __restrict__ image, const ConvGeom& g,
                                                    const int (&hi0)[NV][VEC], const int (&wi0)[NV][VEC], long long k0,
                                                    long long k_rem, int tid) {
    static_assert(!KCONTIG, "the convolution loader walks output pixels fastest");
    const int khw = g.kernel_h * g.kernel_w;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      int x, kk;
      coords(i, tid, x, kk);
      const int kg = static_cast<int>(k0) + kk;
      const int c_id = kg / khw;
      const int k2 = kg - c_id * khw;
      int kh_id = k2 / g.kernel_w;
      int kw_id = k2 - kh_id * g.kernel_w;
      if (g.flip) {
        kh_id = g.kernel_h - 1 - kh_id;
        kw_id = g.kernel_w - 1 - kw_id;
      }
      const int dh = kh_id * g.dil_h;
      const int dw = kw_id * g.dil_w;
      const T* plane = image + static_cast<long long>(c_id) * g.height * g.width;
      const bool k_ok = kk < k_rem;
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const int hi = hi0[i][j] + dh;
        const int wi = wi0[i][j] + dw;
        T val = Tr::st(Tr::zero());
        if (k_ok && hi >= 0 && hi < g.height && wi >= 0 && wi < g.width) val = plane[hi * g.width + wi];
        reg[i][j] = val;
      }
    }
  }

  template <int LDS>
  static __device__ __forceinline__ void stash(S* __restrict__ sm, const T (&reg)[NV][VEC], bool conjugate, int tid) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      int x, kk;
      coords(i, tid, x, kk);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        S v = Tr::ld(reg[i][j]);
        if (conjugate) v = Tr::conj(v);
        if (KCONTIG) {
          sm[(kk + j) * LDS + x] = v;
        } else {
          sm[kk * LDS + x + j] = v;
        }
      }
    }
  }
};

// ---- the kernel -----------------------------------------------------------------------------------------

// GROUPS > 1 lets one CTA work on several tiles at once, each tile owned by a group of (BM/TM)*(BN/TN) threads:
// small batched problems then get a large register tile per thread (high FMA-to-load ratio) and a CTA that is
// still big enough to keep many loads in flight.
template <typename Tr, int BM, int BN, int BK, int TM, int TN, bool A_KC, bool B_KC, bool CONV, int MINB, int GROUPS>
__global__ void __launch_bounds__((BM / TM) * (BN / TN) * GROUPS, MINB)
gemm_simt_kernel(const SimtParams<typename Tr::S> p) {
  using T = typename Tr::T;
  using S = typename Tr::S;
  constexpr int NT = (BM / TM) * (BN / TN);  // threads per tile
  constexpr int CW = Tr::CW;
  constexpr int CWM = (TM < CW) ? TM : CW;  // width of one contiguous chunk of rows owned by a thread
  constexpr int CWN = (TN < CW) ? TN : CW;
  constexpr int NCM = TM / CWM;
  constexpr int NCN = TN / CWN;
  constexpr int PAD = 4;
  constexpr int LDA_S = BM + PAD;
  constexpr int LDB_S = BN + PAD;
  using StA = TileStager<Tr, BM, BK, NT, A_KC>;
  using StB = TileStager<Tr, BN, BK, NT, B_KC>;

  // Dynamic shared memory (configurations above 48 KB need the opt-in attribute the launcher sets):
  // [GROUPS][2][BK * LDA_S] for A followed by [GROUPS][2][BK * LDB_S] for B.
  extern __shared__ __align__(16) unsigned char simt_smem[];
  using ATiles = S[2][BK * LDA_S];
  using BTiles = S[2][BK * LDB_S];
  ATiles* const sA_all = reinterpret_cast<ATiles*>(simt_smem);
  BTiles* const sB_all = reinterpret_cast<BTiles*>(simt_smem + sizeof(ATiles) * GROUPS);

  const int group = (GROUPS > 1) ? threadIdx.x / NT : 0;
  const int tid = (GROUPS > 1) ? threadIdx.x % NT : threadIdx.x;
  S(*sA)[BK * LDA_S] = sA_all[group];
  S(*sB)[BK * LDB_S] = sB_all[group];
  const int tx = tid % (BM / TM);
  const int ty = tid / (BM / TM);
  const bool a_vec_ok = (p.lda % Tr::VEC) == 0;
  const bool b_vec_ok = (p.ldb % Tr::VEC) == 0;

  for (long long first = static_cast<long long>(blockIdx.x) * GROUPS; first < p.total_tiles;
       first += static_cast<long long>(gridDim.x) * GROUPS) {
    // A group without a tile in the last round keeps walking through the barriers on a clamped tile and only
    // skips the stores.
    const bool active = first + group < p.total_tiles;
    const long long tile = active ? first + group : p.total_tiles - 1;
    const long long tm = tile % p.tiles_m;
    const long long rest = tile / p.tiles_m;
    const long long tn = rest % p.tiles_n;
    const long long bz = rest / p.tiles_n;
    const long long m0 = tm * BM, n0 = tn * BN;
    // A tile wholly outside the triangle of a rank-k update is not computed when the CTA owns a single tile (the
    // branch is then uniform over the CTA); in a CTA of several tiles it is computed and all its stores are masked.
    const bool outside = (p.tri == 1 && m0 > n0 + BN - 1) || (p.tri == 2 && n0 > m0 + BM - 1);
    if (GROUPS == 1 && outside) continue;
    const long long m_rem = p.m - m0, n_rem = (active && !outside) ? p.n - n0 : 0;  // n_rem == 0 masks every store
    const bool on_diagonal = p.tri != 0 && m0 < n0 + BN && n0 < m0 + BM;  // element-wise mask needed

    const T* a_base = static_cast<const T*>(p.a) + (p.a_offs ? p.a_offs[bz] : p.a_off + bz * p.a_stride);
    const T* b_base = static_cast<const T*>(p.b) + (p.b_offs ? p.b_offs[bz] : p.b_off + bz * p.b_stride);
    T* c_base = static_cast<T*>(p.c) + (p.c_offs ? p.c_offs[bz] : p.c_off + bz * p.c_stride);
    const S alpha = p.alphas ? p.alphas[bz] : p.alpha;
    const S beta = p.betas ? p.betas[bz] : p.beta;

    S acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = Tr::zero();

    T ra[StA::NV][Tr::VEC];
    T rb[StB::NV][Tr::VEC];

    int conv_h0[CONV ? StA::NV : 1][CONV ? Tr::VEC : 1];
    int conv_w0[CONV ? StA::NV : 1][CONV ? Tr::VEC : 1];
    if constexpr (CONV) StA::conv_pixels(conv_h0, conv_w0, p.conv, m0, m_rem, tid);

    auto fetch_tiles = [&](long long k0) {
      if constexpr (CONV) {
        StA::fetch_conv(ra, a_base, p.conv, conv_h0, conv_w0, k0, p.k - k0, tid);
      } else {
        StA::fetch(ra, a_base, p.lda, m0, k0, m_rem, p.k - k0, a_vec_ok, tid);
      }
      StB::fetch(rb, b_base, p.ldb, n0, k0, p.n - n0, p.k - k0, b_vec_ok, tid);
    };

    fetch_tiles(0);
    __syncthreads();  // previous tile's readers are done with both shared buffers
    StA::template stash<LDA_S>(sA[0], ra, p.conj_a != 0, tid);
    StB::template stash<LDB_S>(sB[0], rb, p.conj_b != 0, tid);
    __syncthreads();

    int cur = 0;
    for (long long k0 = 0; k0 < p.k; k0 += BK) {
      const bool has_next = (k0 + BK) < p.k;
      if (has_next) fetch_tiles(k0 + BK);

      const S* __restrict__ As = sA[cur];
      const S* __restrict__ Bs = sB[cur];
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        S av[TM], bv[TN];
#pragma unroll
        for (int cm = 0; cm < NCM; ++cm) {
          const VecOf<S, CWM> va =
              *reinterpret_cast<const VecOf<S, CWM>*>(&As[kk * LDA_S + cm * (BM / NCM) + tx * CWM]);
#pragma unroll
          for (int i = 0; i < CWM; ++i) av[cm * CWM + i] = va.v[i];
        }
#pragma unroll
        for (int cn = 0; cn < NCN; ++cn) {
          const VecOf<S, CWN> vb =
              *reinterpret_cast<const VecOf<S, CWN>*>(&Bs[kk * LDB_S + cn * (BN / NCN) + ty * CWN]);
#pragma unroll
          for (int j = 0; j < CWN; ++j) bv[cn * CWN + j] = vb.v[j];
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) Tr::mad(acc[i][j], av[i], bv[j]);
      }

      if (has_next) {
        StA::template stash<LDA_S>(sA[cur ^ 1], ra, p.conj_a != 0, tid);
        StB::template stash<LDB_S>(sB[cur ^ 1], rb, p.conj_b != 0, tid);
        __syncthreads();
        cur ^= 1;
      }
    }

    // Epilogue: alpha*acc (+ beta*c). C is only read when beta != 0.
    const bool use_beta = !Tr::is_zero(beta);
    const bool c_vec_ok = (p.ldc % CWM) == 0 && (reinterpret_cast<uintptr_t>(c_base + m0) % (CWM * sizeof(T))) == 0;
#pragma unroll
    for (int cn = 0; cn < NCN; ++cn) {
#pragma unroll
      for (int j = 0; j < CWN; ++j) {
        const long long nn = cn * (BN / NCN) + ty * CWN + j;
        if (nn >= n_rem) continue;
        T* c_col = c_base + (n0 + nn) * p.ldc + m0;
#pragma unroll
        for (int cm = 0; cm < NCM; ++cm) {
          const int mm = cm * (BM / NCM) + tx * CWM;
          if (c_vec_ok && !on_diagonal && mm + CWM <= m_rem) {
            VecOf<T, CWM> out;
            if (use_beta) {
              const VecOf<T, CWM> old = *reinterpret_cast<const VecOf<T, CWM>*>(c_col + mm);
#pragma unroll
              for (int i = 0; i < CWM; ++i)
                out.v[i] = Tr::st(Tr::axpby(alpha, acc[cm * CWM + i][cn * CWN + j], beta, Tr::ld(old.v[i])));
            } else {
#pragma unroll
              for (int i = 0; i < CWM; ++i) out.v[i] = Tr::st(Tr::mul(alpha, acc[cm * CWM + i][cn * CWN + j]));
            }
            *reinterpret_cast<VecOf<T, CWM>*>(c_col + mm) = out;
          } else {
#pragma unroll
            for (int i = 0; i < CWM; ++i) {
              if (mm + i < m_rem) {
                const long long gi = m0 + mm + i, gj = n0 + nn;
                if (on_diagonal && (p.tri == 1 ? gi > gj : gi < gj)) continue;
                const S r = acc[cm * CWM + i][cn * CWN + j];
                S v = use_beta ? Tr::axpby(alpha, r, beta, Tr::ld(c_col[mm + i])) : Tr::mul(alpha, r);
                if (p.real_diag && gi == gj) v = Tr::real_only(v);
                c_col[mm + i] = Tr::st(v);
              }
            }
          }
        }
      }
    }
  }
}

// ---- host-side launch -----------------------------------------------------------------------------------

template <typename Tr, int BM, int BN, int BK, int TM, int TN, int MINB, int GROUPS = 1>
struct SimtLauncher {
  using S = typename Tr::S;

  template <bool A_KC, bool B_KC, bool CONV>
  static cudaError_t go(const GemmDesc& d, cudaStream_t stream) {
    SimtParams<S> p;
    p.a = d.a; p.b = d.b; p.c = d.c;
    p.m = d.m; p.n = d.n; p.k = d.k;
    p.lda = d.lda; p.ldb = d.ldb; p.ldc = d.ldc;
    p.a_off = d.a_off; p.b_off = d.b_off; p.c_off = d.c_off;
    p.a_stride = d.a_stride; p.b_stride = d.b_stride; p.c_stride = d.c_stride;
    p.a_offs = d.a_offs; p.b_offs = d.b_offs; p.c_offs = d.c_offs;
    p.alphas = static_cast<const S*>(d.alphas);
    p.betas = static_cast<const S*>(d.betas);
    p.alpha = Tr::from_host(d.alpha);
    p.beta = Tr::from_host(d.beta);
    p.batch = d.batch;
    p.tiles_m = (d.m + BM - 1) / BM;
    p.tiles_n = (d.n + BN - 1) / BN;
    p.total_tiles = p.tiles_m * p.tiles_n * d.batch;
    p.conj_a = d.conj_a; p.conj_b = d.conj_b;
    p.tri = d.tri; p.real_diag = d.real_diag;
    p.conv = d.conv;
    const long long max_grid = 1LL << 30;
    const long long ctas = (p.total_tiles + GROUPS - 1) / GROUPS;
    const unsigned grid = static_cast<unsigned>(ctas < max_grid ? ctas : max_grid);
    constexpr int NT = (BM / TM) * (BN / TN) * GROUPS;
    constexpr size_t SMEM = sizeof(S) * 2 * BK * ((BM + 4) + (BN + 4)) * GROUPS;
    auto kernel = gemm_simt_kernel<Tr, BM, BN, BK, TM, TN, A_KC, B_KC, CONV, MINB, GROUPS>;
    if (SMEM > 48 * 1024) {  // per-context opt-in (remembered per context)
      const cudaError_t e = kernel_ready(reinterpret_cast<const void*>(kernel), static_cast<int>(SMEM));
      if (e != cudaSuccess) return e;
    }
    kernel<<<grid, NT, SMEM, stream>>>(p);
    return cudaGetLastError();
  }

  static cudaError_t launch_conv(const GemmDesc& d, cudaStream_t stream) { return go<false, true, true>(d, stream); }

  static cudaError_t launch(const GemmDesc& d, cudaStream_t stream) {
    if (d.a_kcontig) {
      return d.b_kcontig ? go<true, true, false>(d, stream) : go<true, false, false>(d, stream);
    }
    return d.b_kcontig ? go<false, true, false>(d, stream) : go<false, false, false>(d, stream);
  }
};

}  // namespace b200
