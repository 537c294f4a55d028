/* C ABI of the B200 GEMM library (libclblast.so).
 *
 * One flat extern "C" entry point per routine of CLBlast's GEMM family. The C++ templates of
 * include/clblast_cuda.h are thin shims over these; other languages bind these directly.
 * Conventions shared by all entry points:
 *   - `dtype` is CLBlast's Precision value: 16 (IEEE half), 32, 64, 3232 (complex float), 6464 (complex double).
 *   - `layout`, `a_transpose`, `b_transpose`, `kernel_mode` are CLBlast's enum values (101/102, 111/112/113, 151/152).
 *   - matrices are DEVICE pointers; offsets, leading dimensions and strides are in elements of the dtype.
 *   - scalars are passed by HOST pointer to one element of the dtype (half: a 16-bit pattern; complex: re, im).
 *   - the return value is CLBlast's StatusCode as an int: 0 success, negative CLBlast codes, positive CUresult.
 *   - `async == 0` reproduces the reference's semantics: the work runs on a library-owned non-blocking stream
 *     and the call returns after it completed (`stream` is ignored). `async != 0` enqueues the work on `stream`
 *     (a CUstream / cudaStream_t, NULL being the default stream) and returns without waiting.
 *   - nothing is ever computed on the host: if no sm_100 device is usable the call fails with a CUresult.
 * The caller's CUDA context must be current on the calling thread.
 */
#ifndef B200BLAS_H_
#define B200BLAS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces clblast::Gemm<T> (reference: include/clblast_cuda.h:385-390, src/clblast_cuda.cpp:1158-1178,
 * host logic src/routines/level3/xgemm.cpp:57-94). */
int b200blas_gemm(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n, size_t k,
                  const void* alpha, const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset,
                  size_t b_ld, const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async);

/* Replaces clblast::GemmStridedBatched<T> (include/clblast_cuda.h:511-518, src/clblast_cuda.cpp:1763-1783,
 * src/routines/levelx/xgemmstridedbatched.cpp:59-102). */
int b200blas_gemm_strided_batched(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n,
                                  size_t k, const void* alpha, const void* a, size_t a_offset, size_t a_ld,
                                  size_t a_stride, const void* b, size_t b_offset, size_t b_ld, size_t b_stride,
                                  const void* beta, void* c, size_t c_offset, size_t c_ld, size_t c_stride,
                                  size_t batch_count, void* stream, int async);

/* Replaces clblast::GemmBatched<T> (include/clblast_cuda.h:502-507, src/clblast_cuda.cpp:1704-1734,
 * src/routines/levelx/xgemmbatched.cpp:59-112). `alphas`, `betas` and the three offset arrays are HOST arrays
 * of batch_count entries; the library stages them into device scratch it owns. */
int b200blas_gemm_batched(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n, size_t k,
                          const void* alphas, const void* a, const size_t* a_offsets, size_t a_ld, const void* b,
                          const size_t* b_offsets, size_t b_ld, const void* betas, void* c, const size_t* c_offsets,
                          size_t c_ld, size_t batch_count, void* stream, int async);

/* GemmBatched without any device allocation. It has no counterpart in the reference, whose GemmBatched allocates
 * and uploads five device arrays per call (src/routines/levelx/xgemmbatched.cpp:87-90,255-260).
 * For programs that cannot allocate device memory when they call: processes whose own arena already owns all of
 * the GPU's memory, and latency-critical loops that must stay clear of the allocator's locks and implicit
 * synchronisation. The per-batch offset and scalar tables go into a fixed array inside the library image instead
 * of allocator scratch. Same arguments, checks and results as b200blas_gemm_batched, except:
 *   - batch_count may not exceed B200BLAS_STATIC_MAX_BATCHES (kInvalidBatchCount, -2049, otherwise);
 *   - the work is always enqueued on the caller's `stream`; `wait != 0` synchronises that stream before returning;
 *   - all calls on one GPU share the array (about 224 KB per GPU, held until the process exits) and it keeps the
 *     last call's tables, so calls that could overlap on the GPU (other streams, other threads) must be ordered
 *     by the caller;
 *   - the first call under each CUDA context resolves the array's device address in that context;
 *   - a stream that is being captured is refused with kUnexpectedError (-2039) before anything is enqueued: the
 *     host block that the table copy reads is reused by the next call;
 *   - with `wait != 0` an expired bounded wait of a tensor-core kernel is reported as kUnexpectedError, as the
 *     regular entry point does; with `wait == 0` use b200blas_tensor_core_status after synchronising. */
#define B200BLAS_STATIC_MAX_BATCHES 4096
int b200blas_gemm_batched_static(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n,
                                 size_t k, const void* alphas, const void* a, const size_t* a_offsets, size_t a_ld,
                                 const void* b, const size_t* b_offsets, size_t b_ld, const void* betas, void* c,
                                 const size_t* c_offsets, size_t c_ld, size_t batch_count, void* stream, int wait);

/* Replaces clblast::Convgemm<T> (include/clblast_cuda.h:486-493, src/clblast_cuda.cpp:1625-1645,
 * src/routines/levelx/xconvgemm.cpp:50-161). dtype 16, 32 or 64. */
int b200blas_convgemm(int dtype, int kernel_mode, size_t channels, size_t height, size_t width, size_t kernel_h,
                      size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w,
                      size_t dilation_h, size_t dilation_w, size_t num_kernels, size_t batch_count, const void* im,
                      size_t im_offset, const void* kernel, size_t kernel_offset, void* result, size_t result_offset,
                      void* stream, int async);

/* ---- level-3 routines built on the GEMM path -------------------------------------------------------------------
 * `side` 141/142 (left/right), `triangle` 121/122 (upper/lower), `diagonal` 131/132 (non-unit/unit): CLBlast's enum
 * values. Scratch (a square copy of the triangular operand, a copy of B, inverted diagonal blocks) comes from the
 * stream-ordered allocator and is released in stream order. */

/* Replace clblast::Symm<T> / Hemm<T>: C = alpha*A*B + beta*C (left) or alpha*B*A + beta*C (right), A symmetric /
 * hermitian with one triangle stored (include/clblast_cuda.h:393-406, src/clblast_cuda.cpp:1199-1266,
 * src/routines/level3/xsymm.cpp:33-96, xhemm.cpp:33-96). Hemm: dtype 3232 or 6464. */
int b200blas_symm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha, const void* a,
                  size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld, const void* beta, void* c,
                  size_t c_offset, size_t c_ld, void* stream, int async);
int b200blas_hemm(int dtype, int layout, int side, int triangle, size_t m, size_t n, const void* alpha, const void* a,
                  size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld, const void* beta, void* c,
                  size_t c_offset, size_t c_ld, void* stream, int async);

/* Replace clblast::Syrk<T> / Herk<T>: the `triangle` of C = alpha*A*A^T + beta*C (a_transpose 111) or
 * alpha*A^T*A + beta*C (include/clblast_cuda.h:409-420, src/clblast_cuda.cpp:1269-1327,
 * src/routines/level3/xsyrk.cpp:51-160, xherk.cpp:51-165). Herk: dtype 3232 / 6464, conjugate transposes, alpha and
 * beta point to REAL scalars (float / double), the diagonal of C comes out real. */
int b200blas_syrk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k, const void* alpha,
                  const void* a, size_t a_offset, size_t a_ld, const void* beta, void* c, size_t c_offset, size_t c_ld,
                  void* stream, int async);
int b200blas_herk(int dtype, int layout, int triangle, int a_transpose, size_t n, size_t k, const void* alpha,
                  const void* a, size_t a_offset, size_t a_ld, const void* beta, void* c, size_t c_offset, size_t c_ld,
                  void* stream, int async);

/* Replace clblast::Syr2k<T> / Her2k<T,U>: the `triangle` of C = alpha*A*B^T + alpha*B*A^T + beta*C, or with both
 * operands transposed (include/clblast_cuda.h:423-436, src/clblast_cuda.cpp:1330-1397,
 * src/routines/level3/xsyr2k.cpp:33-50, xher2k.cpp:33-52). Her2k: alpha complex, beta points to a REAL scalar,
 * C = alpha*A*B^H + conj(alpha)*B*A^H + beta*C. */
int b200blas_syr2k(int dtype, int layout, int triangle, int ab_transpose, size_t n, size_t k, const void* alpha,
                   const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                   const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async);
int b200blas_her2k(int dtype, int layout, int triangle, int ab_transpose, size_t n, size_t k, const void* alpha,
                   const void* a, size_t a_offset, size_t a_ld, const void* b, size_t b_offset, size_t b_ld,
                   const void* beta, void* c, size_t c_offset, size_t c_ld, void* stream, int async);

/* Replaces clblast::Trmm<T>: B = alpha*op(A)*B (left) or alpha*B*op(A) (right), A triangular
 * (include/clblast_cuda.h:439-443, src/clblast_cuda.cpp:1400-1436, src/routines/level3/xtrmm.cpp:33-110). */
int b200blas_trmm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m, size_t n,
                  const void* alpha, const void* a, size_t a_offset, size_t a_ld, void* b, size_t b_offset, size_t b_ld,
                  void* stream, int async);

/* Replaces clblast::Trsm<T>: solves op(A)*X = alpha*B (left) or X*op(A) = alpha*B (right) for X, which overwrites B
 * (include/clblast_cuda.h:446-450, src/clblast_cuda.cpp:1439-1471, src/routines/level3/xtrsm.cpp:40-243,
 * src/routines/levelx/xinvert.cpp:42-150). dtype 32, 64, 3232 or 6464. */
int b200blas_trsm(int dtype, int layout, int side, int triangle, int a_transpose, int diagonal, size_t m, size_t n,
                  const void* alpha, const void* a, size_t a_offset, size_t a_ld, void* b, size_t b_offset, size_t b_ld,
                  void* stream, int async);

/* ---- the copies either side of the GEMM path --------------------------------------------------------------------- */

/* Replaces clblast::Omatcopy<T>: B = alpha*op(A), out of place (include/clblast_cuda.h:464-467,
 * src/clblast_cuda.cpp:1510-1544, src/routines/levelx/xomatcopy.cpp:45-78). */
int b200blas_omatcopy(int dtype, int layout, int a_transpose, size_t m, size_t n, const void* alpha, const void* a,
                      size_t a_offset, size_t a_ld, void* b, size_t b_offset, size_t b_ld, void* stream, int async);

/* Replace clblast::Im2col<T> / Col2im<T> for one image [channels][height][width] and its column matrix
 * [channels * kernel_h * kernel_w][output_h * output_w] (include/clblast_cuda.h:470-483,
 * src/clblast_cuda.cpp:1547-1623, src/routines/levelx/xim2col.cpp:38-95, xcol2im.cpp:38-105). Col2im ADDS the
 * gathered sums to the image, as the reference does. */
int b200blas_im2col(int dtype, int kernel_mode, size_t channels, size_t height, size_t width, size_t kernel_h,
                    size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w, size_t dilation_h,
                    size_t dilation_w, const void* im, size_t im_offset, void* col, size_t col_offset, void* stream,
                    int async);
int b200blas_col2im(int dtype, int kernel_mode, size_t channels, size_t height, size_t width, size_t kernel_h,
                    size_t kernel_w, size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w, size_t dilation_h,
                    size_t dilation_w, const void* col, size_t col_offset, void* im, size_t im_offset, void* stream,
                    int async);

/* Replaces clblast::GemmTempBufferSize<T> (include/clblast_cuda.h:523-527, src/clblast_cuda.cpp:1818-1843).
 * Validates the dimensions and writes 0: no kernel of this library needs caller scratch. */
int b200blas_gemm_temp_buffer_size(int dtype, int layout, int a_transpose, int b_transpose, size_t m, size_t n,
                                   size_t k, size_t a_offset, size_t a_ld, size_t b_offset, size_t b_ld,
                                   size_t c_offset, size_t c_ld, size_t* temp_buffer_size);

/* Replace clblast::ClearCache / FillCache (include/clblast_cuda.h:533-537, src/api_common.cpp:25-33,120-135). */
int b200blas_clear_cache(void);
int b200blas_fill_cache(int device);

/* Replace clblast::OverrideParameters / RetrieveParameters (include/clblast_cuda.h:541-550,
 * src/api_common.cpp:140-221) with a flat form: `names` is an array of `count` NUL-terminated strings and
 * `values` the matching numbers. Retrieve writes at most `capacity` entries (names are pointers to storage
 * owned by the library, valid until the next override of that family) and stores the family's size in *count. */
int b200blas_override_parameters(int device, const char* kernel_name, int precision, const char* const* names,
                                 const size_t* values, size_t count);
int b200blas_retrieve_parameters(int device, const char* kernel_name, int precision, const char** names,
                                 size_t* values, size_t capacity, size_t* count);

/* Limits how many SMs the persistent tensor-core kernels occupy (0 = all, the default). A caller that overlaps a
 * GEMM with a collective or a copy kernel on another stream leaves those a few SMs this way. Process-wide.
 * No counterpart in the reference. */
void b200blas_set_sm_budget(int sms);

/* Multi-GPU building blocks (no counterpart in the reference, which is a single-device library). The sharded GEMM
 * needs the operand that is not split on every GPU; these calls move it with the copy engines, so that no collective
 * kernel competes with the persistent GEMM kernels for SMs. Kernels of this library only ever read local memory.
 *   b200blas_ipc_export: 64-byte handle of the device allocation that contains `device_ptr`, plus the pointer's
 *     byte offset inside it; another process of the same node maps it with b200blas_ipc_open (peer access is
 *     enabled on demand) and unmaps it with b200blas_ipc_close(pointer, offset).
 *   b200blas_stream_copy: cudaMemcpyAsync with the direction inferred from the pointers; `dst` may be a mapped
 *     peer pointer. One call per copy.
 *   b200blas_stream_wait_flag: work enqueued on `stream` after this call starts once the 32-bit word at `flag`
 *     (LOCAL device memory, 4-byte aligned) is >= `value`; no SM is occupied while waiting. The writer is a peer's
 *     4-byte b200blas_stream_copy into that word, ordered after the payload copy on the peer's stream.
 *   b200blas_stream_write_flag: stream-ordered store of `value` to a 32-bit word in local device memory.
 * All return 0 or a CUDA error number. */
int b200blas_ipc_export(const void* device_ptr, unsigned char handle[64], size_t* offset);
int b200blas_ipc_open(const unsigned char handle[64], size_t offset, void** device_ptr);
int b200blas_ipc_close(void* device_ptr, size_t offset);
int b200blas_stream_copy(void* stream, void* dst, const void* src, size_t bytes);
int b200blas_stream_wait_flag(void* stream, const void* flag, uint32_t value);
int b200blas_stream_write_flag(void* stream, void* flag, uint32_t value);

/* The tensor-core kernels bound every wait on a barrier; a wait that expires (a lost copy, a defect) makes the
 * kernel leave a code in a status block and return instead of hanging. Synchronous calls check the block themselves
 * and return kUnexpectedError. Callers that enqueue on their own stream (`async != 0`) call this after that stream
 * has been synchronised: it copies the block (code, block index, barrier address, 0) to `out` (may be NULL), clears
 * it when `clear != 0`, and returns 0 when no wait has expired since the last clear, kUnexpectedError otherwise.
 * No counterpart in the reference. */
int b200blas_tensor_core_status(unsigned int out[4], int clear);

/* Introspection for tests and benchmarks (no counterpart in the reference). */

/* Name of the kernel family the selection table picked for the most recent compute call on this thread,
 * e.g. "tc_f16_128x256", "simt_128x128", "simt_32x32", "conv_simt". Never NULL. */
const char* b200blas_last_kernel(void);
/* Number of kernel launches issued by this library in this process so far. */
uint64_t b200blas_launch_count(void);
/* Library version string. */
const char* b200blas_version(void);

#ifdef __cplusplus
}
#endif

#endif /* B200BLAS_H_ */
