// The level-3 routines that sit on the GEMM path, and the copy / im2col routines either side of it.
//
// Host logic mirrored from the reference (behaviour, not code):
//   Symm / Hemm / Trmm: the triangle is expanded to a square matrix, then one GEMM (src/routines/level3/xsymm.cpp:33-96,
//     xhemm.cpp:33-96, xtrmm.cpp:33-110; Trmm multiplies a copy of B into B);
//   Syrk / Herk / Syr2k / Her2k: one or two GEMMs whose result is written to one triangle of C only
//     (xsyrk.cpp:51-160, xherk.cpp:51-165, xsyr2k.cpp:33-50, xher2k.cpp:33-52);
//   Trsm: inverses of the diagonal blocks, then block substitution built from GEMMs (xtrsm.cpp:40-243); here the
//     blocks are 64 wide and the substitution is recursive, so most of the arithmetic sits in large GEMMs;
//   Omatcopy / Im2col / Col2im: xomatcopy.cpp:45-78, xim2col.cpp:38-95, xcol2im.cpp:38-105.
// Scratch (the square copy, the copy of B, the block inverses) comes from the stream-ordered allocator and is released
// in stream order; everything is enqueued on one stream without host synchronisation in between.
#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstdio>

#include "b200blas.h"
#include "host_common.h"
#include "kernels/level3_aux.h"

namespace b200 {

namespace {

// Stream-ordered scratch released when the scope ends (in stream order, so the kernels enqueued before still own it).
struct Scratch {
  void* ptr = nullptr;
  cudaStream_t stream = nullptr;
  cudaError_t get(size_t bytes, cudaStream_t s) {
    stream = s;
    return cudaMallocAsync(&ptr, bytes, s);
  }
  ~Scratch() {
    if (ptr) cudaFreeAsync(ptr, stream);
  }
};

const double kOne[2] = {1.0, 0.0}, kZero[2] = {0.0, 0.0}, kMinusOne[2] = {-1.0, 0.0};

bool valid_triangle(int t) { return t == kUpper || t == kLower; }
bool valid_side(int s) { return s == kLeft || s == kRight; }
bool valid_transpose(int t) { return t == kNo || t == kYes || t == kConjugate; }
bool valid_layout(int l) { return l == kRowMajor || l == kColMajor; }

int cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return kSuccess;
  std::fprintf(stderr, "b200blas: CUDA error %d (%s)\n", static_cast<int>(e), cudaGetErrorString(e));
  cudaGetLastError();
  return static_cast<int>(e);
}

// Symm (kind 0) and Hemm (kind 1).
int symm_like(int kind, int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha,
              const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
              const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_layout(layout) || !valid_side(side) || !valid_triangle(triangle) || !alpha || !beta)
    return kUnexpectedError;
  if (kind == 1 && dtype < 100) return kNotImplemented;
  if (m == 0 || n == 0) return kInvalidDimension;
  const size_t k = (side == kLeft) ? m : n;
  int st = test_matrix(k, k, a, a_offset, a_ld, elem, true, kInvalidLeadDimA, kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  const size_t one = (layout == kRowMajor) ? n : m, two = (layout == kRowMajor) ? m : n;
  st = test_matrix(one, two, b, b_offset, b_ld, elem, true, kInvalidLeadDimB, kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  st = test_matrix(one, two, c, c_offset, c_ld, elem, true, kInvalidLeadDimC, kInsufficientMemoryC, kInvalidMatrixC);
  if (st) return st;
  double al[2], be[2];
  read_scalar(dtype, alpha, 0, al);
  read_scalar(dtype, beta, 0, be);
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  Scratch square;
  cudaError_t err = square.get(k * k * elem, s);
  if (err != cudaSuccess) return cuda_status(err);
  // the kernels see memory order: a row-major upper triangle is a column-major lower one
  const bool mem_upper = (triangle == kUpper) != (layout == kRowMajor);
  err = launch_densify(dtype, kind, mem_upper, false, static_cast<long long>(k), a, static_cast<long long>(a_offset),
                       static_cast<long long>(a_ld), square.ptr, s);
  if (err != cudaSuccess) return cuda_status(err);
  st = (side == kLeft)
           ? gemm_enqueue(dtype, layout, kNo, kNo, m, n, k, al, square.ptr, 0, k, b, b_offset, b_ld, be, c, c_offset,
                          c_ld, s)
           : gemm_enqueue(dtype, layout, kNo, kNo, m, n, k, al, b, b_offset, b_ld, square.ptr, 0, k, be, c, c_offset,
                          c_ld, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

// Transposes of the two operands of one triangle-masked product of the rank-k family (SyrkAB / HerkAB of the
// reference): the second operand gets the opposite transpose; the hermitian forms conjugate.
void rank_k_transposes(bool hermitian, int ab_transpose, int* ta, int* tb) {
  *ta = ab_transpose;
  *tb = (ab_transpose != kNo) ? kNo : kYes;
  if (hermitian) {
    *ta = (*ta != kNo) ? kConjugate : kNo;
    *tb = (*tb != kNo) ? kConjugate : kNo;
  }
}

int rank_k_validate(int dtype, bool hermitian, int layout, int ab_transpose, size_t n, size_t k, const void* a,
                    size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld, const void* c,
                    size_t c_offset, size_t c_ld) {
  int ta, tb;
  rank_k_transposes(hermitian, ab_transpose, &ta, &tb);
  return gemm_validate(dtype, layout, ta, tb, n, n, k, a, a_offset, a_ld, b, b_offset, b_ld, c, c_offset, c_ld);
}

// C = alpha * op(A) * op(B) + beta * C on one triangle; with `real_diag` the diagonal of C is kept real.
int rank_k_product(int dtype, bool hermitian, int layout, int triangle, int ab_transpose, size_t n, size_t k,
                   const double alpha[2], const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset,
                   size_t b_ld, const double beta[2], void* c, size_t c_offset, size_t c_ld, bool real_diag,
                   cudaStream_t s) {
  int ta, tb;
  rank_k_transposes(hermitian, ab_transpose, &ta, &tb);
  return gemm_enqueue(dtype, layout, ta, tb, n, n, k, alpha, a, a_offset, a_ld, b, b_offset, b_ld, beta, c, c_offset,
                      c_ld, s, triangle, real_diag ? 1 : 0);
}

// ---- Trsm ---------------------------------------------------------------------------------------------------------

constexpr size_t kTrsmBlock = 64;

struct TrsmPlan {
  int dtype;
  bool left, forward;  // forward: block 0 is solved first
  int a_transpose;
  size_t m, n, k;
  const void* a; size_t a_offset, a_ld;
  void* b; size_t b_offset, b_ld;   // receives X
  void* w; size_t w_ld;             // working right-hand side (alpha * B, updated as blocks are eliminated)
  const void* inv;                  // inverted diagonal blocks
  cudaStream_t stream;
};

// Element offset of op(A)(r0, c0) in the caller's A.
size_t sub_a(const TrsmPlan& p, size_t r0, size_t c0) {
  return p.a_offset + (p.a_transpose == kNo ? r0 + c0 * p.a_ld : c0 + r0 * p.a_ld);
}

int trsm_base(const TrsmPlan& p, size_t block) {
  const size_t i0 = block * kTrsmBlock, bs = std::min(kTrsmBlock, p.k - i0);
  const size_t inv_off = block * kTrsmBlock * kTrsmBlock;
  if (p.left) {  // X_i = op(inv_i) * W_i
    return gemm_enqueue(p.dtype, kColMajor, p.a_transpose, kNo, bs, p.n, bs, kOne, p.inv, inv_off, kTrsmBlock, p.w, i0,
                        p.w_ld, kZero, p.b, p.b_offset + i0, p.b_ld, p.stream);
  }
  // X_j = W_j * op(inv_j)
  return gemm_enqueue(p.dtype, kColMajor, kNo, p.a_transpose, p.m, bs, bs, kOne, p.w, i0 * p.w_ld, p.w_ld, p.inv,
                      inv_off, kTrsmBlock, kZero, p.b, p.b_offset + i0 * p.b_ld, p.b_ld, p.stream);
}

// Solves the block range [lo, hi): one half, then the other half's right-hand side is updated with one large GEMM.
int trsm_range(const TrsmPlan& p, size_t lo, size_t hi) {
  if (hi - lo == 1) return trsm_base(p, lo);
  const size_t mid = lo + (hi - lo) / 2;
  const size_t e0 = lo * kTrsmBlock, e1 = mid * kTrsmBlock, e2 = std::min(hi * kTrsmBlock, p.k);
  const size_t first = e1 - e0, second = e2 - e1;
  int st = p.forward ? trsm_range(p, lo, mid) : trsm_range(p, mid, hi);
  if (st != kSuccess) return st;
  if (p.left && p.forward) {         // W[second] -= op(A)[second, first] * X[first]
    st = gemm_enqueue(p.dtype, kColMajor, p.a_transpose, kNo, second, p.n, first, kMinusOne, p.a, sub_a(p, e1, e0), p.a_ld,
                      p.b, p.b_offset + e0, p.b_ld, kOne, p.w, e1, p.w_ld, p.stream);
  } else if (p.left) {               // W[first] -= op(A)[first, second] * X[second]
    st = gemm_enqueue(p.dtype, kColMajor, p.a_transpose, kNo, first, p.n, second, kMinusOne, p.a, sub_a(p, e0, e1), p.a_ld,
                      p.b, p.b_offset + e1, p.b_ld, kOne, p.w, e0, p.w_ld, p.stream);
  } else if (p.forward) {            // W[:, second] -= X[:, first] * op(A)[first, second]
    st = gemm_enqueue(p.dtype, kColMajor, kNo, p.a_transpose, p.m, second, first, kMinusOne, p.b, p.b_offset + e0 * p.b_ld,
                      p.b_ld, p.a, sub_a(p, e0, e1), p.a_ld, kOne, p.w, e1 * p.w_ld, p.w_ld, p.stream);
  } else {                           // W[:, first] -= X[:, second] * op(A)[second, first]
    st = gemm_enqueue(p.dtype, kColMajor, kNo, p.a_transpose, p.m, first, second, kMinusOne, p.b, p.b_offset + e1 * p.b_ld,
                      p.b_ld, p.a, sub_a(p, e1, e0), p.a_ld, kOne, p.w, e0 * p.w_ld, p.w_ld, p.stream);
  }
  if (st != kSuccess) return st;
  return p.forward ? trsm_range(p, mid, hi) : trsm_range(p, lo, mid);
}

int conv_geometry(size_t channels, size_t height, size_t width, size_t kernel_h, size_t kernel_w, size_t pad_h,
                  size_t pad_w, size_t stride_h, size_t stride_w, size_t dilation_h, size_t dilation_w, int kernel_mode,
                  ConvGeom* g, size_t* out_h) {
  if (kernel_mode != kCrossCorrelation && kernel_mode != kConvolution) return kUnexpectedError;
  if (channels == 0 || height == 0 || width == 0) return kInvalidDimension;
  if (kernel_h == 0 || kernel_w == 0 || stride_h == 0 || stride_w == 0 || dilation_h == 0 || dilation_w == 0)
    return kInvalidDimension;
  const size_t size_h = height + 2 * pad_h, padding_h = dilation_h * (kernel_h - 1) + 1;
  const size_t size_w = width + 2 * pad_w, padding_w = dilation_w * (kernel_w - 1) + 1;
  *out_h = (size_h >= padding_h) ? (size_h - padding_h) / stride_h + 1 : 1;
  const size_t out_w = (size_w >= padding_w) ? (size_w - padding_w) / stride_w + 1 : 1;
  const size_t int_max = 0x7FFFFFFF;
  if (channels * height * width > int_max || kernel_h * kernel_w > int_max || *out_h * out_w > int_max ||
      pad_h > int_max || pad_w > int_max || stride_h > int_max || stride_w > int_max || dilation_h > int_max ||
      dilation_w > int_max)
    return kInvalidDimension;
  g->channels = static_cast<int>(channels); g->height = static_cast<int>(height); g->width = static_cast<int>(width);
  g->kernel_h = static_cast<int>(kernel_h); g->kernel_w = static_cast<int>(kernel_w);
  g->pad_h = static_cast<int>(pad_h); g->pad_w = static_cast<int>(pad_w);
  g->stride_h = static_cast<int>(stride_h); g->stride_w = static_cast<int>(stride_w);
  g->dil_h = static_cast<int>(dilation_h); g->dil_w = static_cast<int>(dilation_w);
  g->out_w = static_cast<int>(out_w);
  g->flip = (kernel_mode == kConvolution);
  return kSuccess;
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" int b200blas_symm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha,
                             const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                             const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async) {
  return symm_like(0, dtype, layout, side, triangle, m, n, alpha, a, a_offset, a_ld, b, b_offset, b_ld, beta, c, c_offset,
                   c_ld, stream, async);
}

extern "C" int b200blas_hemm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha,
                             const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                             const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async) {
  return symm_like(1, dtype, layout, side, triangle, m, n, alpha, a, a_offset, a_ld, b, b_offset, b_ld, beta, c, c_offset,
                   c_ld, stream, async);
}

extern "C" int b200blas_syrk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k, const void* alpha,
                             const void* a, size_t a_offset, size_t a_ld, const void* beta, void* c, size_t c_offset,
                             size_t c_ld, void* stream, int async) {
  if (dtype_size(dtype) == 0 || !valid_layout(layout) || !valid_triangle(triangle) || !valid_transpose(a_transpose) ||
      !alpha || !beta)
    return kUnexpectedError;
  double al[2], be[2];
  read_scalar(dtype, alpha, 0, al);
  read_scalar(dtype, beta, 0, be);
  int st = rank_k_validate(dtype, false, layout, a_transpose, n, k, a, a_offset, a_ld, a, a_offset, a_ld, c, c_offset, c_ld);
  if (st != kSuccess) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  st = rank_k_product(dtype, false, layout, triangle, a_transpose, n, k, al, a, a_offset, a_ld, a, a_offset, a_ld, be, c,
                      c_offset, c_ld, false, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_herk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k, const void* alpha,
                             const void* a, size_t a_offset, size_t a_ld, const void* beta, void* c, size_t c_offset,
                             size_t c_ld, void* stream, int async) {
  if ((dtype != 3232 && dtype != 6464) || !valid_layout(layout) || !valid_triangle(triangle) ||
      !valid_transpose(a_transpose) || !alpha || !beta)
    return dtype_size(dtype) != 0 && dtype < 100 ? kNotImplemented : kUnexpectedError;
  // alpha and beta are real scalars of the matching real precision
  double al[2] = {0.0, 0.0}, be[2] = {0.0, 0.0};
  read_scalar(dtype == 3232 ? 32 : 64, alpha, 0, al);
  read_scalar(dtype == 3232 ? 32 : 64, beta, 0, be);
  int st = rank_k_validate(dtype, true, layout, a_transpose, n, k, a, a_offset, a_ld, a, a_offset, a_ld, c, c_offset, c_ld);
  if (st != kSuccess) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  st = rank_k_product(dtype, true, layout, triangle, a_transpose, n, k, al, a, a_offset, a_ld, a, a_offset, a_ld, be, c,
                      c_offset, c_ld, true, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_syr2k(int dtype, int layout, int triangle, int ab_transpose, size_t n, size_t k,
                              const void* alpha, const void* a, size_t a_offset, size_t a_ld, const void* b,
                              size_t b_offset, size_t b_ld, const void* beta, void* c, size_t c_offset, size_t c_ld,
                              void* stream, int async) {
  if (dtype_size(dtype) == 0 || !valid_layout(layout) || !valid_triangle(triangle) || !valid_transpose(ab_transpose) ||
      !alpha || !beta)
    return kUnexpectedError;
  double al[2], be[2];
  read_scalar(dtype, alpha, 0, al);
  read_scalar(dtype, beta, 0, be);
  int st = rank_k_validate(dtype, false, layout, ab_transpose, n, k, a, a_offset, a_ld, b, b_offset, b_ld, c, c_offset, c_ld);
  if (st != kSuccess) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  // C = alpha*A*B^T + beta*C, then C = alpha*B*A^T + C, both on the triangle only
  st = rank_k_product(dtype, false, layout, triangle, ab_transpose, n, k, al, a, a_offset, a_ld, b, b_offset, b_ld, be, c,
                      c_offset, c_ld, false, s);
  if (st != kSuccess) return st;
  st = rank_k_product(dtype, false, layout, triangle, ab_transpose, n, k, al, b, b_offset, b_ld, a, a_offset, a_ld, kOne,
                      c, c_offset, c_ld, false, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_her2k(int dtype, int layout, int triangle, int ab_transpose, size_t n, size_t k,
                              const void* alpha, const void* a, size_t a_offset, size_t a_ld, const void* b,
                              size_t b_offset, size_t b_ld, const void* beta, void* c, size_t c_offset, size_t c_ld,
                              void* stream, int async) {
  if ((dtype != 3232 && dtype != 6464) || !valid_layout(layout) || !valid_triangle(triangle) ||
      !valid_transpose(ab_transpose) || !alpha || !beta)
    return dtype_size(dtype) != 0 && dtype < 100 ? kNotImplemented : kUnexpectedError;
  double al[2], be[2] = {0.0, 0.0};
  read_scalar(dtype, alpha, 0, al);                           // complex
  read_scalar(dtype == 3232 ? 32 : 64, beta, 0, be);          // real
  const double conj_al[2] = {al[0], -al[1]};
  int st = rank_k_validate(dtype, true, layout, ab_transpose, n, k, a, a_offset, a_ld, b, b_offset, b_ld, c, c_offset, c_ld);
  if (st != kSuccess) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  // C = alpha*A*B^H + beta*C, then C = conj(alpha)*B*A^H + C with the diagonal made real
  st = rank_k_product(dtype, true, layout, triangle, ab_transpose, n, k, al, a, a_offset, a_ld, b, b_offset, b_ld, be, c,
                      c_offset, c_ld, false, s);
  if (st != kSuccess) return st;
  st = rank_k_product(dtype, true, layout, triangle, ab_transpose, n, k, conj_al, b, b_offset, b_ld, a, a_offset, a_ld,
                      kOne, c, c_offset, c_ld, true, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_trmm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m,
                             size_t n, const void* alpha, const void* a, size_t a_offset, size_t a_ld, void* b,
                             size_t b_offset, size_t b_ld, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_layout(layout) || !valid_side(side) || !valid_triangle(triangle) ||
      !valid_transpose(a_transpose) || (diagonal != kUnit && diagonal != kNonUnit) || !alpha)
    return kUnexpectedError;
  if (m == 0 || n == 0) return kInvalidDimension;
  const size_t k = (side == kLeft) ? m : n;
  int st = test_matrix(k, k, a, a_offset, a_ld, elem, true, kInvalidLeadDimA, kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  const size_t b_one = (layout == kRowMajor) ? n : m, b_two = (layout == kRowMajor) ? m : n;
  st = test_matrix(b_one, b_two, b, b_offset, b_ld, elem, true, kInvalidLeadDimB, kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  double al[2];
  read_scalar(dtype, alpha, 0, al);
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  // the product cannot overwrite its own input: B is multiplied from a copy (same leading dimension, offset 0)
  const size_t b_elems = b_ld * (b_two - 1) + b_one;
  Scratch square, b_copy;
  cudaError_t err = square.get(k * k * elem, s);
  if (err == cudaSuccess) err = b_copy.get(b_elems * elem, s);
  if (err == cudaSuccess)
    err = cudaMemcpyAsync(b_copy.ptr, static_cast<const unsigned char*>(b) + b_offset * elem, b_elems * elem,
                          cudaMemcpyDeviceToDevice, s);
  const bool mem_upper = (triangle == kUpper) != (layout == kRowMajor);
  if (err == cudaSuccess)
    err = launch_densify(dtype, 2, mem_upper, diagonal == kUnit, static_cast<long long>(k), a,
                         static_cast<long long>(a_offset), static_cast<long long>(a_ld), square.ptr, s);
  if (err != cudaSuccess) return cuda_status(err);
  st = (side == kLeft)
           ? gemm_enqueue(dtype, layout, a_transpose, kNo, m, n, k, al, square.ptr, 0, k, b_copy.ptr, 0, b_ld, kZero, b,
                          b_offset, b_ld, s)
           : gemm_enqueue(dtype, layout, kNo, a_transpose, m, n, k, al, b_copy.ptr, 0, b_ld, square.ptr, 0, k, kZero, b,
                          b_offset, b_ld, s);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_trsm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m,
                             size_t n, const void* alpha, const void* a, size_t a_offset, size_t a_ld, void* b,
                             size_t b_offset, size_t b_ld, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_layout(layout) || !valid_side(side) || !valid_triangle(triangle) ||
      !valid_transpose(a_transpose) || (diagonal != kUnit && diagonal != kNonUnit) || !alpha)
    return kUnexpectedError;
  if (dtype == 16) return kNotImplemented;  // the reference has no half-precision Trsm either
  // A row-major problem is the column-major problem with the other side and the other triangle (B' = X' A').
  if (layout == kRowMajor) {
    std::swap(m, n);
    side = (side == kLeft) ? kRight : kLeft;
    triangle = (triangle == kLower) ? kUpper : kLower;
  }
  if (m == 0 || n == 0) return kInvalidDimension;
  const size_t k = (side == kLeft) ? m : n;
  int st = test_matrix(k, k, a, a_offset, a_ld, elem, true, kInvalidLeadDimA, kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(m, n, b, b_offset, b_ld, elem, true, kInvalidLeadDimB, kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  double al[2];
  read_scalar(dtype, alpha, 0, al);
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;

  const size_t blocks = (k + kTrsmBlock - 1) / kTrsmBlock;
  Scratch work, inverses;
  cudaError_t err = work.get(m * n * elem, s);
  if (err == cudaSuccess) err = inverses.get(blocks * kTrsmBlock * kTrsmBlock * elem, s);
  // W = alpha * B, compact
  if (err == cudaSuccess)
    err = launch_omatcopy(dtype, false, false, static_cast<long long>(m), static_cast<long long>(n), al, b,
                          static_cast<long long>(b_offset), static_cast<long long>(b_ld), work.ptr, 0,
                          static_cast<long long>(m), s);
  if (err == cudaSuccess)
    err = launch_invert_diagonal_blocks(dtype, triangle == kUpper, diagonal == kUnit, static_cast<long long>(k),
                                        static_cast<int>(kTrsmBlock), a, static_cast<long long>(a_offset),
                                        static_cast<long long>(a_ld), inverses.ptr, s);
  if (err != cudaSuccess) return cuda_status(err);

  TrsmPlan p;
  p.dtype = dtype;
  p.left = (side == kLeft);
  // op(A) is lower triangular when (lower, not transposed) or (upper, transposed): a left solve then runs from the
  // first block down, a right solve from the last block up.
  const bool op_lower = (triangle == kUpper) != (a_transpose == kNo);
  p.forward = p.left ? op_lower : !op_lower;
  p.a_transpose = a_transpose;
  p.m = m; p.n = n; p.k = k;
  p.a = a; p.a_offset = a_offset; p.a_ld = a_ld;
  p.b = b; p.b_offset = b_offset; p.b_ld = b_ld;
  p.w = work.ptr; p.w_ld = m;
  p.inv = inverses.ptr;
  p.stream = s;
  st = trsm_range(p, 0, blocks);
  if (st != kSuccess) return st;
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_omatcopy(int dtype, int layout, int a_transpose, size_t m, size_t n, const void* alpha,
                                 const void* a, size_t a_offset, size_t a_ld, void* b, size_t b_offset, size_t b_ld,
                                 void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0 || !valid_layout(layout) || !valid_transpose(a_transpose) || !alpha) return kUnexpectedError;
  if (m == 0 || n == 0) return kInvalidDimension;
  const bool transpose = a_transpose != kNo;
  const size_t a_one = (layout == kRowMajor) ? n : m, a_two = (layout == kRowMajor) ? m : n;
  const size_t b_one = transpose ? a_two : a_one, b_two = transpose ? a_one : a_two;
  int st = test_matrix(a_one, a_two, a, a_offset, a_ld, elem, true, kInvalidLeadDimA, kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(b_one, b_two, b, b_offset, b_ld, elem, true, kInvalidLeadDimB, kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  double al[2];
  read_scalar(dtype, alpha, 0, al);
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  const cudaError_t err =
      launch_omatcopy(dtype, transpose, a_transpose == kConjugate, static_cast<long long>(a_one),
                      static_cast<long long>(a_two), al, a, static_cast<long long>(a_offset),
                      static_cast<long long>(a_ld), b, static_cast<long long>(b_offset), static_cast<long long>(b_ld), s);
  if (err != cudaSuccess) return cuda_status(err);
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_im2col(int dtype, int kernel_mode, size_t channels, size_t height, size_t width, size_t kernel_h,
                               size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w,
                               size_t dilation_h, size_t dilation_w, const void* im, size_t im_offset, void* col,
                               size_t col_offset, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0) return kUnexpectedError;
  ConvGeom g;
  size_t out_h = 0;
  int st = conv_geometry(channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h,
                         dilation_w, kernel_mode, &g, &out_h);
  if (st) return st;
  st = test_matrix(channels * height * width, 1, im, im_offset, channels * height * width, elem, false, kInvalidLeadDimA,
                   kInsufficientMemoryA, kInvalidMatrixA);
  if (st) return st;
  const size_t col_elems = channels * kernel_h * kernel_w * out_h * static_cast<size_t>(g.out_w);
  st = test_matrix(col_elems, 1, col, col_offset, col_elems, elem, false, kInvalidLeadDimB, kInsufficientMemoryB,
                   kInvalidMatrixB);
  if (st) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  const cudaError_t err = launch_im2col(dtype, g, static_cast<int>(out_h), im, static_cast<long long>(im_offset), col,
                                        static_cast<long long>(col_offset), s);
  if (err != cudaSuccess) return cuda_status(err);
  return end_call(s, async, cudaSuccess);
}

extern "C" int b200blas_col2im(int dtype, int kernel_mode, size_t channels, size_t height, size_t width, size_t kernel_h,
                               size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w,
                               size_t dilation_h, size_t dilation_w, const void* col, size_t col_offset, void* im,
                               size_t im_offset, void* stream, int async) {
  const size_t elem = dtype_size(dtype);
  if (elem == 0) return kUnexpectedError;
  ConvGeom g;
  size_t out_h = 0;
  int st = conv_geometry(channels, height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dilation_h,
                         dilation_w, kernel_mode, &g, &out_h);
  if (st) return st;
  const size_t col_elems = channels * kernel_h * kernel_w * out_h * static_cast<size_t>(g.out_w);
  st = test_matrix(col_elems, 1, col, col_offset, col_elems, elem, false, kInvalidLeadDimA, kInsufficientMemoryA,
                   kInvalidMatrixA);
  if (st) return st;
  st = test_matrix(channels * height * width, 1, im, im_offset, channels * height * width, elem, false, kInvalidLeadDimB,
                   kInsufficientMemoryB, kInvalidMatrixB);
  if (st) return st;
  cudaStream_t s;
  const int r = begin_call(stream, async, &s);
  if (r != 0) return r;
  const cudaError_t err = launch_col2im(dtype, g, static_cast<int>(out_h), col, static_cast<long long>(col_offset), im,
                                        static_cast<long long>(im_offset), s);
  if (err != cudaSuccess) return cuda_status(err);
  return end_call(s, async, cudaSuccess);
}
