// Internal helpers shared between the C-ABI layer and the allocation-free batched entry point.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>

#include "kernels/gemm_desc.h"

namespace b200 {

// Byte layout of the staged per-batch tables: three offset tables, then alphas, then betas.
struct BatchedTables {
  size_t off_block;
  size_t sc_bytes;
  size_t total;
  size_t batch_count;
};

int prepare_batched(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* alphas,
                    const void* a, const size_t* a_offsets, size_t a_ld, const void* b, const size_t* b_offsets,
                    size_t b_ld, const void* betas, void* c, const size_t* c_offsets, size_t c_ld, size_t batch_count,
                    unsigned char* host_block, size_t host_capacity, GemmDesc* out, BatchedTables* tables);
void patch_batched_tables(GemmDesc* d, const BatchedTables& t, const unsigned char* device_block);
cudaError_t dispatch_desc(const GemmDesc& d, cudaStream_t stream);
// After the stream of a launch has been synchronised: kUnexpectedError when a tensor-core kernel reported an expired
// wait, else 0.
int status_after_sync();

}  // namespace b200
