// Helper kernels around the GEMM path. All of them are bound by HBM bandwidth or are tiny: they move every element
// once with coalesced accesses on both sides (transposing through shared-memory tiles where the two sides disagree).
//
// They replace, for the level-3 routines built on GEMM, the reference's convert / copy / transpose kernels
// (src/kernels/level3/convert_symmetric.opencl, convert_hermitian.opencl, convert_triangular.opencl, copy_pad.opencl,
// transpose_pad.opencl), its diagonal-block inversion (src/kernels/level3/invert_diagonal_blocks_part1.opencl) and the
// im2col / col2im kernels (src/kernels/levelx/im2col.opencl, col2im.opencl).
#include "level3_aux.h"
#include "../runtime_state.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

namespace {

// ---- element arithmetic per storage type -----------------------------------------------------------------------
// S is the type scalars are held in (half data is scaled in fp32 and rounded once, which equals a half multiply).

template <typename T> struct El;
template <> struct El<__half> {
  using S = float;
  static __device__ __forceinline__ __half zero() { return __float2half_rn(0.f); }
  static __device__ __forceinline__ __half one() { return __float2half_rn(1.f); }
  static __device__ __forceinline__ __half conj(__half v) { return v; }
  static __device__ __forceinline__ __half real_only(__half v) { return v; }
  static __device__ __forceinline__ __half scale(S a, __half v) { return __float2half_rn(a * __half2float(v)); }
  static __device__ __forceinline__ __half add(__half a, __half b) { return __hadd(a, b); }
  static __host__ S scalar(const double* v) { return static_cast<float>(v[0]); }
};
template <> struct El<float> {
  using S = float;
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float one() { return 1.f; }
  static __device__ __forceinline__ float conj(float v) { return v; }
  static __device__ __forceinline__ float real_only(float v) { return v; }
  static __device__ __forceinline__ float scale(S a, float v) { return __fmul_rn(a, v); }
  static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
  static __host__ S scalar(const double* v) { return static_cast<float>(v[0]); }
};
template <> struct El<double> {
  using S = double;
  static __device__ __forceinline__ double zero() { return 0.0; }
  static __device__ __forceinline__ double one() { return 1.0; }
  static __device__ __forceinline__ double conj(double v) { return v; }
  static __device__ __forceinline__ double real_only(double v) { return v; }
  static __device__ __forceinline__ double scale(S a, double v) { return __dmul_rn(a, v); }
  static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
  static __host__ S scalar(const double* v) { return v[0]; }
};
template <> struct El<float2> {
  using S = float2;
  static __device__ __forceinline__ float2 zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ float2 one() { return make_float2(1.f, 0.f); }
  static __device__ __forceinline__ float2 conj(float2 v) { return make_float2(v.x, -v.y); }
  static __device__ __forceinline__ float2 real_only(float2 v) { return make_float2(v.x, 0.f); }
  static __device__ __forceinline__ float2 scale(S a, float2 v) {
    return make_float2(a.x * v.x - a.y * v.y, a.x * v.y + a.y * v.x);
  }
  static __device__ __forceinline__ float2 add(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
  static __host__ S scalar(const double* v) { return make_float2(static_cast<float>(v[0]), static_cast<float>(v[1])); }
};
template <> struct El<double2> {
  using S = double2;
  static __device__ __forceinline__ double2 zero() { return make_double2(0.0, 0.0); }
  static __device__ __forceinline__ double2 one() { return make_double2(1.0, 0.0); }
  static __device__ __forceinline__ double2 conj(double2 v) { return make_double2(v.x, -v.y); }
  static __device__ __forceinline__ double2 real_only(double2 v) { return make_double2(v.x, 0.0); }
  static __device__ __forceinline__ double2 scale(S a, double2 v) {
    return make_double2(a.x * v.x - a.y * v.y, a.x * v.y + a.y * v.x);
  }
  static __device__ __forceinline__ double2 add(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }
  static __host__ S scalar(const double* v) { return make_double2(v[0], v[1]); }
};

constexpr int TILE = 32;   // square tiles moved by blocks of 32 x 8 threads
constexpr int ROWS = 8;

template <typename F>
cudaError_t by_dtype(int dtype, F&& f) {
  switch (dtype) {
    case 16: return f(static_cast<__half*>(nullptr));
    case 32: return f(static_cast<float*>(nullptr));
    case 64: return f(static_cast<double*>(nullptr));
    case 3232: return f(static_cast<float2*>(nullptr));
    case 6464: return f(static_cast<double2*>(nullptr));
    default: return cudaErrorInvalidValue;
  }
}

// ---- square matrix from a stored triangle -------------------------------------------------------------------------

// Each block produces one 32 x 32 tile of the result from the same tile of the source and from its mirror image,
// both read along the source's contiguous direction; the mirror tile is transposed through shared memory.
template <typename T, int KIND>
__global__ void __launch_bounds__(TILE * ROWS) densify_kernel(long long k, const T* __restrict__ src, long long ld,
                                                              T* __restrict__ dst, int mem_upper, int unit_diag) {
  __shared__ T own[TILE][TILE + 1];
  __shared__ T mir[TILE][TILE + 1];
  const long long r0 = static_cast<long long>(blockIdx.x) * TILE, c0 = static_cast<long long>(blockIdx.y) * TILE;
  const int x = threadIdx.x;
  for (int y = threadIdx.y; y < TILE; y += ROWS) {
    const long long r = r0 + x, c = c0 + y;
    if (r < k && c < k) own[y][x] = src[c * ld + r];
    const long long mr = c0 + x, mc = r0 + y;  // element (mr, mc) of the source: the mirror of (mc, mr)
    if (KIND != 2 && mr < k && mc < k) mir[y][x] = src[mc * ld + mr];
  }
  __syncthreads();
  for (int y = threadIdx.y; y < TILE; y += ROWS) {
    const long long r = r0 + x, c = c0 + y;
    if (r >= k || c >= k) continue;
    const bool stored = mem_upper ? (r <= c) : (r >= c);
    T v;
    if (stored) {
      v = own[y][x];
      if (KIND == 1 && r == c) v = El<T>::real_only(v);
      if (KIND == 2 && r == c && unit_diag) v = El<T>::one();
    } else if (KIND == 2) {
      v = El<T>::zero();
    } else {
      v = mir[x][y];
      if (KIND == 1) v = El<T>::conj(v);
    }
    dst[c * k + r] = v;
  }
}

// ---- scaled copy / transpose -----------------------------------------------------------------------------------------

template <typename T, bool TRANSPOSE>
__global__ void __launch_bounds__(TILE * ROWS) omatcopy_kernel(long long one, long long two, typename El<T>::S alpha,
                                                               const T* __restrict__ a, long long a_ld,
                                                               T* __restrict__ b, long long b_ld, int conjugate) {
  __shared__ T tile[TILE][TILE + 1];
  const long long x0 = static_cast<long long>(blockIdx.x) * TILE, y0 = static_cast<long long>(blockIdx.y) * TILE;
  const int x = threadIdx.x;
  for (int y = threadIdx.y; y < TILE; y += ROWS) {
    const long long i = x0 + x, j = y0 + y;  // element i of the contiguous direction, line j
    if (i < one && j < two) {
      T v = a[j * a_ld + i];
      if (conjugate) v = El<T>::conj(v);
      v = El<T>::scale(alpha, v);
      if (TRANSPOSE) tile[y][x] = v; else b[j * b_ld + i] = v;
    }
  }
  if (TRANSPOSE) {
    __syncthreads();
    for (int y = threadIdx.y; y < TILE; y += ROWS) {
      const long long j = y0 + x, i = x0 + y;  // the destination is contiguous along the source's lines
      if (i < one && j < two) b[i * b_ld + j] = tile[x][y];
    }
  }
}

// ---- inverses of the diagonal blocks of a triangular matrix -----------------------------------------------------------

template <typename S> struct Arith;
template <> struct Arith<float> {
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float one() { return 1.f; }
  static __device__ __forceinline__ float neg(float a) { return -a; }
  static __device__ __forceinline__ float fma(float a, float b, float c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ float inv(float a) { return 1.f / a; }
  static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
};
template <> struct Arith<double> {
  static __device__ __forceinline__ double zero() { return 0.0; }
  static __device__ __forceinline__ double one() { return 1.0; }
  static __device__ __forceinline__ double neg(double a) { return -a; }
  static __device__ __forceinline__ double fma(double a, double b, double c) { return ::fma(a, b, c); }
  static __device__ __forceinline__ double inv(double a) { return 1.0 / a; }
  static __device__ __forceinline__ double mul(double a, double b) { return a * b; }
};
template <> struct Arith<float2> {
  static __device__ __forceinline__ float2 zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ float2 one() { return make_float2(1.f, 0.f); }
  static __device__ __forceinline__ float2 neg(float2 a) { return make_float2(-a.x, -a.y); }
  static __device__ __forceinline__ float2 fma(float2 a, float2 b, float2 c) {
    return make_float2(fmaf(a.x, b.x, fmaf(-a.y, b.y, c.x)), fmaf(a.x, b.y, fmaf(a.y, b.x, c.y)));
  }
  static __device__ __forceinline__ float2 inv(float2 a) {
    const float d = a.x * a.x + a.y * a.y;
    return make_float2(a.x / d, -a.y / d);
  }
  static __device__ __forceinline__ float2 mul(float2 a, float2 b) {
    return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
  }
};
template <> struct Arith<double2> {
  static __device__ __forceinline__ double2 zero() { return make_double2(0.0, 0.0); }
  static __device__ __forceinline__ double2 one() { return make_double2(1.0, 0.0); }
  static __device__ __forceinline__ double2 neg(double2 a) { return make_double2(-a.x, -a.y); }
  static __device__ __forceinline__ double2 fma(double2 a, double2 b, double2 c) {
    return make_double2(::fma(a.x, b.x, ::fma(-a.y, b.y, c.x)), ::fma(a.x, b.y, ::fma(a.y, b.x, c.y)));
  }
  static __device__ __forceinline__ double2 inv(double2 a) {
    const double d = a.x * a.x + a.y * a.y;
    return make_double2(a.x / d, -a.y / d);
  }
  static __device__ __forceinline__ double2 mul(double2 a, double2 b) {
    return make_double2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
  }
};

// One block per diagonal block, one thread per column of the inverse: column j of X = T^-1 follows from T X = I by
// substitution, downwards from the diagonal for a lower triangle, upwards for an upper one. Shared memory holds the
// block as [row][column + pad] so that the threads (columns) of a warp read X conflict-free and T by broadcast.
template <typename T, int NB>
__global__ void __launch_bounds__(NB) invert_blocks_kernel(long long k, const T* __restrict__ a, long long ld,
                                                           T* __restrict__ inv, int mem_upper, int unit_diag) {
  using A = Arith<T>;
  extern __shared__ __align__(16) unsigned char inv_smem[];
  T(*t)[NB + 1] = reinterpret_cast<T(*)[NB + 1]>(inv_smem);
  T(*x)[NB + 1] = t + NB;
  const long long base = static_cast<long long>(blockIdx.x) * NB;
  const int j = threadIdx.x;
  for (int r = 0; r < NB; ++r) {  // thread j loads column j: rows are contiguous in memory, so a warp's loads of one
    const long long gr = base + r, gc = base + j;  // row index hit 32 different lines; the block is tiny and read once
    const bool stored = mem_upper ? (r <= j) : (r >= j);
    T v = (r == j) ? A::one() : A::zero();
    if (stored && gr < k && gc < k && !(r == j && unit_diag)) v = a[gc * ld + gr];
    t[r][j] = v;
    x[r][j] = A::zero();
  }
  __syncthreads();
  if (!mem_upper) {
    x[j][j] = A::inv(t[j][j]);
    for (int i = j + 1; i < NB; ++i) {
      T s = A::zero();
      for (int p = j; p < i; ++p) s = A::fma(t[i][p], x[p][j], s);
      x[i][j] = A::mul(A::neg(s), A::inv(t[i][i]));
    }
  } else {
    x[j][j] = A::inv(t[j][j]);
    for (int i = j - 1; i >= 0; --i) {
      T s = A::zero();
      for (int p = i + 1; p <= j; ++p) s = A::fma(t[i][p], x[p][j], s);
      x[i][j] = A::mul(A::neg(s), A::inv(t[i][i]));
    }
  }
  __syncthreads();
  T* out = inv + static_cast<long long>(blockIdx.x) * NB * NB;
  for (int c = 0; c < NB; ++c) out[c * NB + j] = x[j][c];  // thread j writes row j: consecutive threads, consecutive addresses
}

// ---- im2col / col2im ----------------------------------------------------------------------------------------------------

// One CTA writes one row (channel, kernel index) of one image's column matrix, or several whole rows when a row is
// shorter than the CTA: the row's tap is decoded once per thread, and each thread walks its output pixels with
// additions only. blockIdx.x: row group, blockIdx.y: image (strided when there are more images than grid rows).
template <typename T>
__global__ void __launch_bounds__(256) im2col_kernel(ConvGeom g, int out_h, int plane, int rows_per_cta, int rows,
                                                     long long images, const T* __restrict__ im_all,
                                                     long long im_stride, T* __restrict__ col) {
  const int khw = g.kernel_h * g.kernel_w;
  const int tid = static_cast<int>(threadIdx.x);
  const int local = rows_per_cta > 1 ? tid / plane : 0;
  const int first = rows_per_cta > 1 ? tid - local * plane : tid;
  const int step = rows_per_cta > 1 ? plane : 256;  // several rows per CTA: one element per thread
  const int row = static_cast<int>(blockIdx.x) * rows_per_cta + local;
  if (local >= rows_per_cta || row >= rows) return;
  const int c = row / khw;
  const int kidx = row - c * khw;
  const int tap = g.flip ? khw - 1 - kidx : kidx;  // the tap whose value lands at this kernel index
  const int kh = tap / g.kernel_w, kw = tap - kh * g.kernel_w;
  const int dh = kh * g.dil_h - g.pad_h, dw = kw * g.dil_w - g.pad_w;
  // A thread's pixels are `step` apart: step_h rows and step_w columns further, one more row on a wrap. Row, column and
  // offset inside the channel plane of the tap it reads move by constants, so the loop body is additions and compares.
  const int step_h = step / g.out_w, step_w = step - step_h * g.out_w;
  const int ho0 = first / g.out_w, wo0 = first - ho0 * g.out_w;
  const int h_step = step_h * g.stride_h, w_step = step_w * g.stride_w;
  const int off_step = h_step * g.width + w_step;
  const int w_wrap = g.out_w * g.stride_w, off_wrap = g.stride_h * g.width - w_wrap;
  for (long long image_index = blockIdx.y; image_index < images; image_index += gridDim.y) {
    const T* __restrict__ im = im_all + image_index * im_stride + static_cast<long long>(c) * g.height * g.width;
    T* __restrict__ out = col + (image_index * rows + row) * plane;  // column matrices of consecutive images are adjacent
    int wo = wo0;
    int h = ho0 * g.stride_h + dh, w = wo0 * g.stride_w + dw;
    int off = h * g.width + w;
    // eight pixels per round: all loads are issued before the first store, so eight of them are in flight per thread
    for (int pos0 = first; pos0 < plane; pos0 += 8 * step) {
      T v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = El<T>::zero();
        if (pos0 + i * step < plane && static_cast<unsigned>(h) < static_cast<unsigned>(g.height) &&
            static_cast<unsigned>(w) < static_cast<unsigned>(g.width))
          v[i] = im[off];
        h += h_step; w += w_step; off += off_step; wo += step_w;
        if (wo >= g.out_w) { wo -= g.out_w; w -= w_wrap; h += g.stride_h; off += off_wrap; }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (pos0 + i * step < plane) out[pos0 + i * step] = v[i];
    }
  }
}

// One thread per image pixel gathers, in the reference's order (taps from the last kernel row and column to the
// first), the column entries im2col would have read from that pixel, and adds the sum to the pixel.
template <typename T>
__global__ void col2im_kernel(ConvGeom g, int out_h, long long total, const T* __restrict__ col, T* __restrict__ im) {
  const int khw = g.kernel_h * g.kernel_w;
  const long long plane = static_cast<long long>(out_h) * g.out_w;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int w = static_cast<int>(idx % g.width);
    const long long rest = idx / g.width;
    const int h = static_cast<int>(rest % g.height);
    const int c = static_cast<int>(rest / g.height);
    T sum = El<T>::zero();
    bool any = false;
    for (int kh = g.kernel_h - 1; kh >= 0; --kh) {
      const int hs = h + g.pad_h - kh * g.dil_h;
      if (hs < 0 || hs % g.stride_h != 0) continue;
      const int ho = hs / g.stride_h;
      if (ho >= out_h) continue;
      for (int kw = g.kernel_w - 1; kw >= 0; --kw) {
        const int ws = w + g.pad_w - kw * g.dil_w;
        if (ws < 0 || ws % g.stride_w != 0) continue;
        const int wo = ws / g.stride_w;
        if (wo >= g.out_w) continue;
        const int tap = kh * g.kernel_w + kw;
        const int kidx = g.flip ? khw - 1 - tap : tap;
        sum = El<T>::add(sum, col[(static_cast<long long>(c) * khw + kidx) * plane + static_cast<long long>(ho) * g.out_w + wo]);
        any = true;
      }
    }
    if (any) im[idx] = El<T>::add(im[idx], sum);
  }
}

unsigned grid_for(long long total, int threads) {
  const long long blocks = (total + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count() > 0 ? sm_count() : 1) * 32;
  return static_cast<unsigned>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// ---- re-pitching copy -------------------------------------------------------------------------------------------------

// Every thread produces two 16-byte vectors of the aligned destination from element loads of the (arbitrarily aligned)
// source: the loads of a warp cover one contiguous run, so every sector is fetched from L2 once, and nothing waits on
// anything else. One CTA covers kSegBytes of one line; both jobs share the launch.
constexpr int kSegBytes = 8192;
struct RepitchParams {
  RepitchJob job[2];
  long long segs_per_line[2];
  long long first_block_of_second;
};

template <typename W>  // W: an unsigned type of the element's width
__global__ void __launch_bounds__(256) repitch_kernel(const RepitchParams p) {
  constexpr int SEG = kSegBytes / static_cast<int>(sizeof(W));
  constexpr int VEC = 16 / static_cast<int>(sizeof(W));
  long long block = blockIdx.x;
  const int which = block >= p.first_block_of_second ? 1 : 0;
  if (which) block -= p.first_block_of_second;
  const RepitchJob& job = p.job[which];
  const long long line = block / p.segs_per_line[which];
  const long long x0 = (block - line * p.segs_per_line[which]) * SEG;
  const W* __restrict__ src = static_cast<const W*>(job.src) + line * job.src_ld + x0;
  W* __restrict__ dst = static_cast<W*>(job.dst) + line * job.dst_pitch + x0;
  const long long valid_ll = job.one - x0, padded_ll = job.dst_pitch - x0;  // source / destination elements from x0 on
  const int valid = static_cast<int>(valid_ll < SEG ? valid_ll : SEG);
  const int padded = static_cast<int>(padded_ll < SEG ? padded_ll : SEG);   // a multiple of VEC
  union Vec { uint4 v; W e[VEC]; };
  Vec r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i0 = (static_cast<int>(threadIdx.x) + 256 * h) * VEC;
#pragma unroll
    for (int j = 0; j < VEC; ++j) r[h].e[j] = (i0 + j < valid) ? src[i0 + j] : W(0);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int i0 = (static_cast<int>(threadIdx.x) + 256 * h) * VEC;
    if (i0 < padded) *reinterpret_cast<uint4*>(dst + i0) = r[h].v;
  }
}

}  // namespace

cudaError_t launch_densify(int dtype, int kind, bool mem_upper, bool unit_diag, long long k, const void* src,
                           long long src_off, long long src_ld, void* dst, cudaStream_t stream) {
  if (k <= 0 || kind < 0 || kind > 2) return cudaErrorInvalidValue;
  const long long tiles = (k + TILE - 1) / TILE;
  if (tiles > 65535) return cudaErrorInvalidValue;
  return by_dtype(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    const dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>(tiles)), block(TILE, ROWS);
    const T* s = static_cast<const T*>(src) + src_off;
    T* d = static_cast<T*>(dst);
    if (kind == 0) densify_kernel<T, 0><<<grid, block, 0, stream>>>(k, s, src_ld, d, mem_upper, unit_diag);
    else if (kind == 1) densify_kernel<T, 1><<<grid, block, 0, stream>>>(k, s, src_ld, d, mem_upper, unit_diag);
    else densify_kernel<T, 2><<<grid, block, 0, stream>>>(k, s, src_ld, d, mem_upper, unit_diag);
    return cudaGetLastError();
  });
}

cudaError_t launch_omatcopy(int dtype, bool transpose, bool conjugate, long long one, long long two,
                            const double alpha[2], const void* a, long long a_off, long long a_ld, void* b,
                            long long b_off, long long b_ld, cudaStream_t stream) {
  if (one <= 0 || two <= 0) return cudaErrorInvalidValue;
  const long long tx = (one + TILE - 1) / TILE, ty = (two + TILE - 1) / TILE;
  if (ty > 65535) return cudaErrorInvalidValue;
  return by_dtype(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    const dim3 grid(static_cast<unsigned>(tx), static_cast<unsigned>(ty)), block(TILE, ROWS);
    const T* s = static_cast<const T*>(a) + a_off;
    T* d = static_cast<T*>(b) + b_off;
    const auto al = El<T>::scalar(alpha);
    if (transpose) omatcopy_kernel<T, true><<<grid, block, 0, stream>>>(one, two, al, s, a_ld, d, b_ld, conjugate);
    else omatcopy_kernel<T, false><<<grid, block, 0, stream>>>(one, two, al, s, a_ld, d, b_ld, conjugate);
    return cudaGetLastError();
  });
}

cudaError_t launch_invert_diagonal_blocks(int dtype, bool mem_upper, bool unit_diag, long long k, int nb, const void* a,
                                          long long a_off, long long a_ld, void* inv, cudaStream_t stream) {
  if (k <= 0 || (nb != 16 && nb != 32 && nb != 64) || dtype == 16) return cudaErrorInvalidValue;
  const unsigned blocks = static_cast<unsigned>((k + nb - 1) / nb);
  return by_dtype(dtype, [&](auto* tag) -> cudaError_t {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    if constexpr (std::is_same<T, __half>::value) {
      return cudaErrorInvalidValue;
    } else {
      const T* s = static_cast<const T*>(a) + a_off;
      T* d = static_cast<T*>(inv);
      auto go = [&](auto kernel, int n) -> cudaError_t {
        const size_t smem = 2 * sizeof(T) * n * (n + 1);
        if (smem > 48 * 1024) {
          const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
          if (e != cudaSuccess) return e;
        }
        kernel<<<blocks, n, smem, stream>>>(k, s, a_ld, d, mem_upper, unit_diag);
        return cudaGetLastError();
      };
      if (nb == 16) return go(invert_blocks_kernel<T, 16>, 16);
      if (nb == 32) return go(invert_blocks_kernel<T, 32>, 32);
      return go(invert_blocks_kernel<T, 64>, 64);
    }
  });
}

cudaError_t launch_im2col(int dtype, const ConvGeom& g, int out_h, const void* im, long long im_off, void* col,
                          long long col_off, cudaStream_t stream, long long images, long long im_stride) {
  const long long rows = static_cast<long long>(g.channels) * g.kernel_h * g.kernel_w;
  const long long plane = static_cast<long long>(out_h) * g.out_w;
  // offsets inside one channel plane, padding and the last partial step included, are kept in 32 bits
  const long long reach = (static_cast<long long>(g.height) + 2LL * (g.pad_h > 0 ? g.pad_h : 0) +
                           static_cast<long long>(g.kernel_h) * g.dil_h + 512LL * g.stride_h) * g.width +
                          static_cast<long long>(g.kernel_w) * g.dil_w + 512LL * g.stride_w + g.pad_w;
  if (rows <= 0 || plane <= 0 || images <= 0 || plane > 0x7FFFFFFF - 256 || rows > 0x7FFFFFFF - 256 ||
      reach > 0x7FFFFFFF)
    return cudaErrorInvalidValue;
  const int rows_per_cta = plane >= 256 ? 1 : static_cast<int>(256 / plane);
  const unsigned groups = static_cast<unsigned>((rows + rows_per_cta - 1) / rows_per_cta);
  const dim3 grid(groups, static_cast<unsigned>(images < 65535 ? images : 65535));
  return by_dtype(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    im2col_kernel<T><<<grid, 256, 0, stream>>>(g, out_h, static_cast<int>(plane), rows_per_cta, static_cast<int>(rows),
                                               images, static_cast<const T*>(im) + im_off, im_stride,
                                               static_cast<T*>(col) + col_off);
    return cudaGetLastError();
  });
}

cudaError_t launch_col2im(int dtype, const ConvGeom& g, int out_h, const void* col, long long col_off, void* im,
                          long long im_off, cudaStream_t stream) {
  const long long total = static_cast<long long>(g.channels) * g.height * g.width;
  if (total <= 0) return cudaErrorInvalidValue;
  return by_dtype(dtype, [&](auto* tag) {
    using T = typename std::remove_pointer<decltype(tag)>::type;
    col2im_kernel<T><<<grid_for(total, 256), 256, 0, stream>>>(g, out_h, total, static_cast<const T*>(col) + col_off,
                                                               static_cast<T*>(im) + im_off);
    return cudaGetLastError();
  });
}

cudaError_t launch_repitch(int elem_bytes, const RepitchJob (&jobs)[2], cudaStream_t stream) {
  if (elem_bytes != 2 && elem_bytes != 4) return cudaErrorInvalidValue;
  const long long seg = kSegBytes / elem_bytes, vec = 16 / elem_bytes;
  RepitchParams p = {};
  long long blocks[2] = {0, 0};
  for (int j = 0; j < 2; ++j) {
    p.job[j] = jobs[j];
    if (jobs[j].two <= 0 || jobs[j].one <= 0) { p.job[j].two = 0; p.segs_per_line[j] = 1; continue; }
    if ((reinterpret_cast<uintptr_t>(jobs[j].dst) & 15) || (jobs[j].dst_pitch % vec) || jobs[j].dst_pitch < jobs[j].one)
      return cudaErrorInvalidValue;
    p.segs_per_line[j] = (jobs[j].dst_pitch + seg - 1) / seg;
    blocks[j] = p.segs_per_line[j] * jobs[j].two;
  }
  p.first_block_of_second = blocks[0];
  const long long total = blocks[0] + blocks[1];
  if (total <= 0) return cudaSuccess;
  if (total > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
  if (elem_bytes == 2) repitch_kernel<unsigned short><<<static_cast<unsigned>(total), 256, 0, stream>>>(p);
  else repitch_kernel<unsigned int><<<static_cast<unsigned>(total), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace b200
