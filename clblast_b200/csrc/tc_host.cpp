#include "tc_host.h"

#include <stdint.h>

#include "driver_api.h"

namespace b200 {

bool encode_operand_map(CUtensorMap* map, int elem_bytes, const void* base, long long rows, long long k, long long ld,
                        bool mn_contig, int kmajor_box_rows, long long batches, long long batch_stride) {
  const DriverApi& drv = driver_api();
  if (!drv.ok) return false;
  const cuuint32_t inner = static_cast<cuuint32_t>(128 / elem_bytes);  // elements per 128-byte swizzle row
  cuuint64_t dims[3];
  cuuint32_t box[3];
  if (mn_contig) {
    dims[0] = static_cast<cuuint64_t>(rows); dims[1] = static_cast<cuuint64_t>(k);
    box[0] = inner; box[1] = inner;
  } else {
    dims[0] = static_cast<cuuint64_t>(k); dims[1] = static_cast<cuuint64_t>(rows);
    box[0] = inner; box[1] = static_cast<cuuint32_t>(kmajor_box_rows);
  }
  dims[2] = static_cast<cuuint64_t>(batches > 1 ? batches : 1);
  box[2] = 1;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(ld) * elem_bytes;
  // a single problem needs no third stride; any legal value will do
  const cuuint64_t batch_bytes = batches > 1 ? static_cast<cuuint64_t>(batch_stride) * elem_bytes : row_bytes;
  if ((row_bytes & 15) || (batch_bytes & 15) || row_bytes >= (1ULL << 40) || batch_bytes >= (1ULL << 40)) return false;
  const cuuint64_t strides[2] = {row_bytes, batch_bytes};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType type = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const CUtensorMapSwizzle swizzle =
      (elem_bytes == 4 && mn_contig) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  return drv.TensorMapEncodeTiled(map, type, 3, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_half_c_map(CUtensorMap* map, const void* base, long long m, long long n, long long ldc, long long batches,
                       long long batch_stride) {
  const DriverApi& drv = driver_api();
  if (!drv.ok) return false;
  if (reinterpret_cast<uintptr_t>(base) & 15) return false;
  const cuuint64_t row_bytes = static_cast<cuuint64_t>(ldc) * 2;
  const cuuint64_t batch_bytes = batches > 1 ? static_cast<cuuint64_t>(batch_stride) * 2 : row_bytes;
  if ((row_bytes & 15) || (batch_bytes & 15) || row_bytes >= (1ULL << 40) || batch_bytes >= (1ULL << 40)) return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(m), static_cast<cuuint64_t>(n),
                              static_cast<cuuint64_t>(batches > 1 ? batches : 1)};
  const cuuint64_t strides[2] = {row_bytes, batch_bytes};
  const cuuint32_t box[3] = {128, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return drv.TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

BatchWalk batch_walk(const GemmDesc& d) {
  BatchWalk w = {};
  if (d.batch < 1 || d.batch > 0x7FFFFFFF) return w;
  if (d.a_offs != nullptr && !d.uniform_strides) return w;  // arbitrary per-problem offsets
  w.batches = static_cast<int>(d.batch);
  if (d.batch == 1) {
    w.a_batches = w.b_batches = 1;
    w.ok = true;
    return w;
  }
  if (d.a_stride < 0 || d.b_stride < 0 || d.c_stride <= 0) return w;
  w.a_stride = d.a_stride;
  w.b_stride = d.b_stride;
  w.c_stride = d.c_stride;
  w.a_batches = d.a_stride == 0 ? 1 : w.batches;
  w.b_batches = d.b_stride == 0 ? 1 : w.batches;
  w.ok = true;
  return w;
}

}  // namespace b200
