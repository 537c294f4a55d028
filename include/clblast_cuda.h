// CLBlast-compatible CUDA API, GEMM family only (B200 / sm_100a implementation).
//
// This header declares the subset of CLBlast's CUDA-flavoured C++ API that this library implements:
// Gemm, GemmBatched, GemmStridedBatched, Convgemm, GemmTempBufferSize and the cache / parameter calls.
// Names, namespaces, enum values, argument order and argument types are those of the reference's
// include/clblast_cuda.h (enums :40-101, Gemm :385-390, Convgemm :486-493, GemmBatched :502-507,
// GemmStridedBatched :511-518, GemmTempBufferSize :523-527, cache/parameter calls :533-550), so the symbols
// exported by libclblast.so have the same Itanium-mangled names and a program compiled against the
// reference's own header links and runs against this library unchanged. Routines outside the GEMM family are
// not declared here and not exported.
//
// All sizes, offsets, leading dimensions and strides are in elements of T. T is float, double,
// unsigned short (IEEE half bit pattern), std::complex<float> or std::complex<double>; Convgemm has no
// complex instantiations. Calls are host-synchronous: the work is complete when the call returns. The
// calling thread must have `context` current, as with the reference.
#ifndef CLBLAST_CLBLAST_CUDA_H_
#define CLBLAST_CLBLAST_CUDA_H_

#include <cstdlib>
#include <string>
#include <unordered_map>

#include <cuda.h>

#ifndef PUBLIC_API
#define PUBLIC_API
#endif

namespace clblast {

// Status codes: 0 is success, negative values are CLBlast codes, positive values are raw CUresult values.
// The numeric values are part of the ABI.
enum class StatusCode {
  kSuccess = 0,
  kInvalidLocalNumDimensions = -53,
  kInvalidLocalThreadsTotal = -54,
  kInvalidLocalThreadsDim = -55,
  kNotImplemented = -1024,
  kInvalidMatrixA = -1022,
  kInvalidMatrixB = -1021,
  kInvalidMatrixC = -1020,
  kInvalidVectorX = -1019,
  kInvalidVectorY = -1018,
  kInvalidDimension = -1017,
  kInvalidLeadDimA = -1016,
  kInvalidLeadDimB = -1015,
  kInvalidLeadDimC = -1014,
  kInvalidIncrementX = -1013,
  kInvalidIncrementY = -1012,
  kInsufficientMemoryA = -1011,
  kInsufficientMemoryB = -1010,
  kInsufficientMemoryC = -1009,
  kInsufficientMemoryX = -1008,
  kInsufficientMemoryY = -1007,
  kInsufficientMemoryTemp = -2050,
  kInvalidBatchCount = -2049,
  kInvalidOverrideKernel = -2048,
  kMissingOverrideParameter = -2047,
  kInvalidLocalMemUsage = -2046,
  kNoHalfPrecision = -2045,
  kNoDoublePrecision = -2044,
  kInvalidVectorScalar = -2043,
  kInsufficientMemoryScalar = -2042,
  kDatabaseError = -2041,
  kUnknownError = -2040,
  kUnexpectedError = -2039,
  kInvalidVectorZ = -2038,
  kInvalidIncrementZ = -2037,
  kInsufficientMemoryZ = -2036,
};

enum class Layout { kRowMajor = 101, kColMajor = 102 };
enum class Transpose { kNo = 111, kYes = 112, kConjugate = 113 };
enum class Triangle { kUpper = 121, kLower = 122 };
enum class Diagonal { kNonUnit = 131, kUnit = 132 };
enum class Side { kLeft = 141, kRight = 142 };
enum class KernelMode { kCrossCorrelation = 151, kConvolution = 152 };
enum class Precision { kHalf = 16, kSingle = 32, kDouble = 64, kComplexSingle = 3232, kComplexDouble = 6464, kAny = -1 };

// C = alpha * op(A) * op(B) + beta * C. With beta == 0 the previous contents of C are never read.
template <typename T>
StatusCode Gemm(const Layout layout, const Transpose a_transpose, const Transpose b_transpose, const size_t m,
                const size_t n, const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset,
                const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice device, CUdeviceptr temp_buffer = 0);

// ---- level-3 routines built on the GEMM path (signatures as in the reference's header) ----------------------------

// C = alpha * A * B + beta * C (side left) or alpha * B * A + beta * C, A symmetric with one triangle stored.
template <typename T>
StatusCode Symm(const Layout layout, const Side side, const Triangle triangle, const size_t m, const size_t n,
                const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice device);

// The same for a hermitian A (complex types).
template <typename T>
StatusCode Hemm(const Layout layout, const Side side, const Triangle triangle, const size_t m, const size_t n,
                const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice device);

// One triangle of C = alpha * A * A^T + beta * C (or A^T * A).
template <typename T>
StatusCode Syrk(const Layout layout, const Triangle triangle, const Transpose a_transpose, const size_t n,
                const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const T beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice device);

// One triangle of C = alpha * A * A^H + beta * C (or A^H * A); T is the real type, the matrices are complex.
template <typename T>
StatusCode Herk(const Layout layout, const Triangle triangle, const Transpose a_transpose, const size_t n,
                const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                const T beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                const CUdevice device);

// One triangle of C = alpha * A * B^T + alpha * B * A^T + beta * C (or with both operands transposed).
template <typename T>
StatusCode Syr2k(const Layout layout, const Triangle triangle, const Transpose ab_transpose, const size_t n,
                 const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                 const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const T beta,
                 CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                 const CUdevice device);

// One triangle of C = alpha * A * B^H + conj(alpha) * B * A^H + beta * C; T complex, U its real type.
template <typename T, typename U>
StatusCode Her2k(const Layout layout, const Triangle triangle, const Transpose ab_transpose, const size_t n,
                 const size_t k, const T alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
                 const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const U beta,
                 CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
                 const CUdevice device);

// B = alpha * op(A) * B (side left) or alpha * B * op(A), A triangular.
template <typename T>
StatusCode Trmm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose,
                const Diagonal diagonal, const size_t m, const size_t n, const T alpha, const CUdeviceptr a_buffer,
                const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset,
                const size_t b_ld, const CUcontext context, const CUdevice device);

// Solves op(A) * X = alpha * B (side left) or X * op(A) = alpha * B; X overwrites B.
template <typename T>
StatusCode Trsm(const Layout layout, const Side side, const Triangle triangle, const Transpose a_transpose,
                const Diagonal diagonal, const size_t m, const size_t n, const T alpha, const CUdeviceptr a_buffer,
                const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t b_offset,
                const size_t b_ld, const CUcontext context, const CUdevice device);

// ---- the copies either side of the GEMM path ------------------------------------------------------------------------

// B = alpha * op(A), out of place.
template <typename T>
StatusCode Omatcopy(const Layout layout, const Transpose a_transpose, const size_t m, const size_t n, const T alpha,
                    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
                    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);

// Column matrix [channels * kernel_h * kernel_w][output_h * output_w] of one image [channels][height][width].
template <typename T>
StatusCode Im2col(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                  const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                  const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                  const CUdeviceptr im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset,
                  const CUcontext context, const CUdevice device);

// The adjoint: adds every column entry to the image pixel it was read from.
template <typename T>
StatusCode Col2im(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                  const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                  const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                  const CUdeviceptr col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset,
                  const CUcontext context, const CUdevice device);

// Batched NCHW convolution expressed as an implicit GEMM; result[n][co][ho][wo], alpha = 1 and beta = 0.
template <typename T>
StatusCode Convgemm(const KernelMode kernel_mode, const size_t channels, const size_t height, const size_t width,
                    const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w,
                    const size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w,
                    const size_t num_kernels, const size_t batch_count, const CUdeviceptr im_buffer,
                    const size_t im_offset, const CUdeviceptr kernel_buffer, const size_t kernel_offset,
                    CUdeviceptr result_buffer, const size_t result_offset, const CUcontext context,
                    const CUdevice device);

// batch_count GEMMs of one shape; per-batch scalars and element offsets are HOST arrays of batch_count entries.
template <typename T>
StatusCode GemmBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose, const size_t m,
                       const size_t n, const size_t k, const T* alphas, const CUdeviceptr a_buffer,
                       const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t* b_offsets,
                       const size_t b_ld, const T* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
                       const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);

// batch_count GEMMs of one shape; batch b uses offset + b * stride for each matrix.
template <typename T>
StatusCode GemmStridedBatched(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                              const size_t m, const size_t n, const size_t k, const T alpha, const CUdeviceptr a_buffer,
                              const size_t a_offset, const size_t a_ld, const size_t a_stride,
                              const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld,
                              const size_t b_stride, const T beta, CUdeviceptr c_buffer, const size_t c_offset,
                              const size_t c_ld, const size_t c_stride, const size_t batch_count,
                              const CUcontext context, const CUdevice device);

// Bytes of caller-provided scratch Gemm would like. This implementation needs none and reports 0.
template <typename T>
StatusCode GemmTempBufferSize(const Layout layout, const Transpose a_transpose, const Transpose b_transpose,
                              const size_t m, const size_t n, const size_t k, const size_t a_offset, const size_t a_ld,
                              const size_t b_offset, const size_t b_ld, const size_t c_offset, const size_t c_ld,
                              const CUdevice device, size_t& temp_buffer_size);

// Kernels are compiled ahead of time, so there is no program cache: both calls succeed and do nothing.
StatusCode PUBLIC_API ClearCache();
StatusCode PUBLIC_API FillCache(const CUdevice device);

// Named tuning parameters are stored and returned but do not change which kernel runs, except
// GemmRoutine/XGEMM_MIN_INDIRECT_SIZE, which is honoured as the size threshold below which the
// small-tile kernel family is forced.
StatusCode PUBLIC_API RetrieveParameters(const CUdevice device, const std::string& kernel_name,
                                         const Precision precision,
                                         std::unordered_map<std::string, size_t>& parameters);
StatusCode PUBLIC_API OverrideParameters(const CUdevice device, const std::string& kernel_name,
                                         const Precision precision,
                                         const std::unordered_map<std::string, size_t>& parameters);

}  // namespace clblast

#endif  // CLBLAST_CLBLAST_CUDA_H_
