// Host-side helpers shared by the tensor-core launchers: tensor maps for operand tiles and the batch geometry.
#pragma once

#include <cuda.h>

#include "kernels/gemm_desc.h"

namespace b200 {

// Tensor map of one GEMM operand, with the batch as third dimension.
//   K-contiguous operand:   dims {K, rows, batches}, box {128 bytes of k, kmajor_box_rows, 1}, 128-byte swizzle.
//   M/N-contiguous operand: dims {rows, K, batches}, box {128 bytes of rows, as many k, 1}; 32-bit elements need the
//   32-byte-chunk flavour of the 128-byte swizzle, which is the only one the tensor cores accept for them.
// elem_bytes is 2 (half) or 4 (float). batch_stride is in elements; with batches == 1 it is ignored.
// Returns false when the driver entry points are missing or the geometry cannot be encoded.
bool encode_operand_map(CUtensorMap* map, int elem_bytes, const void* base, long long rows, long long k, long long ld,
                        bool mn_contig, int kmajor_box_rows, long long batches, long long batch_stride);

// Tensor map for storing a half-precision C (m contiguous): dims {m, n, batches}, box {128 rows, 32 columns, 1}, no
// swizzle (the staging buffer holds 32 columns of 128 contiguous rows). False when C is not 16-byte aligned or its
// leading dimension / batch stride is not a multiple of 8 elements: the caller then stores with plain instructions.
bool encode_half_c_map(CUtensorMap* map, const void* base, long long m, long long n, long long ldc, long long batches,
                       long long batch_stride);

// How a launcher walks the batch of a strided call (or of an offset-table call whose offsets are evenly spaced).
struct BatchWalk {
  bool ok;              // false: the descriptor's batch cannot be expressed with strides
  int batches;          // number of problems
  int a_batches;        // 1 when every problem reads the same A (stride 0), else `batches`
  int b_batches;
  long long a_stride, b_stride, c_stride;  // elements
};
BatchWalk batch_walk(const GemmDesc& d);

}  // namespace b200
