// Normalised, type-erased description of one GEMM-family call, shared by the C-ABI layer and all kernels.
#pragma once

namespace b200 {

// Implicit-GEMM view of a batched NCHW convolution: row p = ho*OW+wo of op(A) and column kk = (c, kh, kw)
// map to image[c][ho*stride_h - pad_h + kh'*dil_h][wo*stride_w - pad_w + kw'*dil_w], zero outside the image;
// (kh', kw') are mirrored when `flip` is set (reference: src/kernels/levelx/xconvgemm_part1.opencl:31-53).
struct ConvGeom {
  int channels, height, width;
  int kernel_h, kernel_w;
  int pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
  int out_w;
  int flip;
};

// Type-erased, normalised problem description handed to every kernel launcher.
struct GemmDesc {
  int dtype;                      // 16, 32, 64, 3232, 6464
  const void* a;
  const void* b;
  void* c;
  long long m, n, k;              // op(A): m x k, op(B): k x n, C: m x n with M contiguous
  long long lda, ldb, ldc;
  long long a_off, b_off, c_off;  // elements
  long long a_stride, b_stride, c_stride;
  const long long* a_offs;        // device tables of per-batch element offsets, or null
  const long long* b_offs;
  const long long* c_offs;
  const void* alphas;             // device tables of per-batch scalars in the kernel's compute type, or null
  const void* betas;
  double alpha[2], beta[2];
  long long batch;
  int a_kcontig, b_kcontig;       // which dimension of each operand has unit stride
  int conj_a, conj_b;
  int is_conv;
  ConvGeom conv;
  int force_small;                // selection-table override: use the small-tile family
  int tables_aligned4;            // every entry of the per-batch offset tables is a multiple of 4 elements
  int uniform_strides;            // the offset tables are evenly spaced: a_off / a_stride etc. describe them too
  // Rank-k updates (Syrk, Herk, Syr2k, Her2k) only write one triangle of the square C: 0 = all of C, 1 = elements
  // with row <= column of the normalised (M-contiguous) C, 2 = elements with row >= column. Tiles wholly outside
  // the triangle are not computed (reference: XgemmUpper / XgemmLower, src/kernels/level3/xgemm_part4.opencl:23-95,
  // and the masked write-back of src/kernels/level3/copy_pad.opencl:100-105).
  int tri;
  int real_diag;                  // Herk / Her2k: the imaginary part of the diagonal of C is set to zero
};

}  // namespace b200
