// Launch interface of the helper kernels around the GEMM path: square matrices from stored triangles, scaled copies
// and transposes, inverses of diagonal blocks, and the im2col / col2im pair.
#pragma once

#include <cuda_runtime_api.h>

#include "gemm_desc.h"

namespace b200 {

// dst (k x k, leading dimension k, element (r, c) at c*k + r) from the triangle of src stored where
// (mem_upper ? r <= c : r >= c), everything in memory order (the caller folds the layout into mem_upper).
// kind 0: symmetric (the other triangle mirrors the stored one); 1: hermitian (mirrored and conjugated, imaginary
// part of the diagonal dropped); 2: triangular (the other triangle is zero; unit_diag puts ones on the diagonal).
// Reference: src/kernels/level3/convert_symmetric.opencl, convert_hermitian.opencl, convert_triangular.opencl.
cudaError_t launch_densify(int dtype, int kind, bool mem_upper, bool unit_diag, long long k, const void* src,
                           long long src_off, long long src_ld, void* dst, cudaStream_t stream);

// b(one x two or, transposed, two x one) = alpha * op(a), `one` being the contiguous extent of a (memory order).
// Reference: PadCopyTransposeMatrix as used by src/routines/levelx/xomatcopy.cpp:73-77.
cudaError_t launch_omatcopy(int dtype, bool transpose, bool conjugate, long long one, long long two,
                            const double alpha[2], const void* a, long long a_off, long long a_ld, void* b,
                            long long b_off, long long b_ld, cudaStream_t stream);

// inv holds ceil(k / nb) dense nb x nb blocks (block i at i*nb*nb, element (r, c) at c*nb + r): the inverses of the
// diagonal blocks of the triangular matrix a (memory order as in launch_densify); the part of the last block beyond
// k is the identity. nb is 16, 32 or 64. Reference: src/routines/levelx/xinvert.cpp:42-150,
// src/kernels/level3/invert_diagonal_blocks_part1.opencl.
cudaError_t launch_invert_diagonal_blocks(int dtype, bool mem_upper, bool unit_diag, long long k, int nb, const void* a,
                                          long long a_off, long long a_ld, void* inv, cudaStream_t stream);

// col[c][kernel index][ho][wo] = im[c][ho*stride - pad + kh*dil][wo*stride - pad + kw*dil] (zero outside the image),
// kernel index = kh*KW + kw, mirrored when g.flip. Reference: src/kernels/levelx/im2col.opencl:24-62.
// `images` > 1: that many images, `im_stride` elements apart; their column matrices follow one another in col.
cudaError_t launch_im2col(int dtype, const ConvGeom& g, int out_h, const void* im, long long im_off, void* col,
                          long long col_off, cudaStream_t stream, long long images = 1, long long im_stride = 0);
// im[c][h][w] += sum of the col entries that im2col would have read from that pixel.
// Reference: src/kernels/levelx/col2im.opencl:29-89.
cudaError_t launch_col2im(int dtype, const ConvGeom& g, int out_h, const void* col, long long col_off, void* im,
                          long long im_off, cudaStream_t stream);

// Copies up to two matrices (`one` contiguous elements per line, `two` lines, any base alignment and leading dimension)
// into destinations whose base is 16-byte aligned and whose pitch is a multiple of 16 bytes, in one launch; the padding
// between `one` and the pitch is zero-filled. Element size 2 or 4 bytes. A job with two == 0 is skipped.
struct RepitchJob {
  const void* src;   // first element
  void* dst;
  long long one, two, src_ld, dst_pitch;  // elements
};
cudaError_t launch_repitch(int elem_bytes, const RepitchJob (&jobs)[2], cudaStream_t stream);

}  // namespace b200
