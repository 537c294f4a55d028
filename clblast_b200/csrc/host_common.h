// Host-side helpers shared by the entry points of the C ABI: status codes, argument checks in the reference's order,
// layout normalisation, the library's private stream and the launch of a normalised problem.
#pragma once

#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>

#include "kernels/gemm_desc.h"

namespace b200 {

// CLBlast status codes used on this path (include/clblast_cuda.h:40-83 of the reference).
enum Status : int {
  kSuccess = 0,
  kNotImplemented = -1024,
  kInvalidMatrixA = -1022,
  kInvalidMatrixB = -1021,
  kInvalidMatrixC = -1020,
  kInvalidDimension = -1017,
  kInvalidLeadDimA = -1016,
  kInvalidLeadDimB = -1015,
  kInvalidLeadDimC = -1014,
  kInsufficientMemoryA = -1011,
  kInsufficientMemoryB = -1010,
  kInsufficientMemoryC = -1009,
  kInvalidBatchCount = -2049,
  kUnknownError = -2040,
  kUnexpectedError = -2039,
};

constexpr int kRowMajor = 101, kColMajor = 102;
constexpr int kNo = 111, kYes = 112, kConjugate = 113;
constexpr int kUpper = 121, kLower = 122;
constexpr int kNonUnit = 131, kUnit = 132;
constexpr int kLeft = 141, kRight = 142;
constexpr int kCrossCorrelation = 151, kConvolution = 152;

size_t dtype_size(int dtype);
// Reads one host scalar of `dtype` into (re, im) doubles.
void read_scalar(int dtype, const void* p, size_t index, double out[2]);

// One matrix check of the reference (src/utilities/buffer_test.hpp:27-73): leading dimension first, then the
// allocation size, with a failing driver query reported as an invalid buffer.
int test_matrix(size_t one, size_t two, const void* buf, size_t offset, size_t ld, size_t elem, bool test_ld,
                int bad_ld, int too_small, int invalid);

struct Extents {
  size_t a_one, a_two, b_one, b_two, c_one, c_two;
  bool a_rotated, b_rotated, c_rotated;
};
// Which dimension of each stored matrix is contiguous (reference: src/routines/level3/xgemm.hpp:87-107).
Extents extents(int layout, int ta, int tb, size_t m, size_t n, size_t k);
bool valid_enums(int layout, int ta, int tb);
void normalise(GemmDesc& d, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* a, size_t a_ld,
               const void* b, size_t b_ld, void* c, size_t c_ld, const Extents& e);
bool force_small_family(int dtype, size_t m, size_t n, size_t k);

// The library-owned non-blocking stream of the current context (one per context, created on first use).
int private_stream(cudaStream_t* out);

// Selects a kernel for the normalised problem and enqueues it on `stream`.
cudaError_t dispatch(const GemmDesc& d, cudaStream_t stream);
// After a synchronous call that ran a tensor-core kernel: kUnexpectedError when a bounded wait expired.
int tensor_core_status(int async);
// Runs `d` either synchronously on the private stream or asynchronously on the caller's stream.
int run(const GemmDesc& d, void* stream, int async);

// The argument checks of one GEMM in the reference's order (dimensions, then A, B, C: leading dimension before size).
int gemm_validate(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* a, size_t a_offset,
                  size_t a_ld, const void* b, size_t b_offset, size_t b_ld, const void* c, size_t c_offset, size_t c_ld);

// One GEMM of the public form, enqueued on `stream` without any synchronisation and without the operand checks
// (callers validate first, before they touch the device). alpha / beta are (re, im). `tri` (0, kUpper or kLower, in
// the caller's layout) and `real_diag` restrict the update to one triangle of C (see GemmDesc).
int gemm_enqueue(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const double alpha[2],
                 const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                 const double beta[2], void* c, size_t c_offset, size_t c_ld, cudaStream_t stream, int tri = 0,
                 int real_diag = 0);

// Picks the stream for an entry point (`async` == 0: the private stream) and finishes it: synchronises when the call
// is synchronous, reports CUDA errors on stderr, checks the tensor-core status block.
int begin_call(void* stream, int async, cudaStream_t* out);
int end_call(cudaStream_t stream, int async, cudaError_t err);

}  // namespace b200
