/* C interface to the device-pointer routines of libclblast.so, named as the reference's C API names them
 * (include/clblast_c.h:885 CLBlastSgemm and its siblings; implementation src/clblast_c.cpp) with the OpenCL handles
 * replaced the way the reference's CUDA header replaces them: matrices are CUdeviceptr, and `cl_command_queue* queue,
 * cl_event* event` becomes `CUcontext context, CUdevice device`. The reference builds its C API for the OpenCL
 * flavour only; this header gives C callers of the CUDA flavour the same names. Every function is host-synchronous
 * and returns a CLBlastStatusCode value (0 success, negative CLBlast codes, positive CUresult values).
 * S / D / C / Z / H: float, double, complex float, complex double, IEEE half (bit pattern). */
#ifndef B200BLAS_C_H_
#define B200BLAS_C_H_

#include <cuda.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int CLBlastStatusCode;
typedef enum CLBlastLayout_ { CLBlastLayoutRowMajor = 101, CLBlastLayoutColMajor = 102 } CLBlastLayout;
typedef enum CLBlastTranspose_ { CLBlastTransposeNo = 111, CLBlastTransposeYes = 112, CLBlastTransposeConjugate = 113 } CLBlastTranspose;
typedef enum CLBlastTriangle_ { CLBlastTriangleUpper = 121, CLBlastTriangleLower = 122 } CLBlastTriangle;
typedef enum CLBlastDiagonal_ { CLBlastDiagonalNonUnit = 131, CLBlastDiagonalUnit = 132 } CLBlastDiagonal;
typedef enum CLBlastSide_ { CLBlastSideLeft = 141, CLBlastSideRight = 142 } CLBlastSide;
typedef enum CLBlastKernelMode_ { CLBlastKernelModeCrossCorrelation = 151, CLBlastKernelModeConvolution = 152 } CLBlastKernelMode;
typedef struct CLBlastComplexFloat_ { float re, im; } CLBlastComplexFloat;
typedef struct CLBlastComplexDouble_ { double re, im; } CLBlastComplexDouble;
typedef unsigned short CLBlastHalf;


/* gemm */
CLBlastStatusCode CLBlastSgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const size_t m, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastDgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const size_t m, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastCgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const
    size_t b_ld, const CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld,
    const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastHgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf alpha, const CUdeviceptr a_buffer,
    const size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld,
    const CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device);

/* symm */
CLBlastStatusCode CLBlastSsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t
    a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const float beta, CUdeviceptr
    c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const double alpha, const CUdeviceptr a_buffer, const size_t a_offset, const
    size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const double beta, CUdeviceptr
    c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastCsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device);
CLBlastStatusCode CLBlastZsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device);
CLBlastStatusCode CLBlastHsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t a_offset, const
    size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CLBlastHalf beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice device);

/* hemm */
CLBlastStatusCode CLBlastChemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device);
CLBlastStatusCode CLBlastZhemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const size_t m, const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device);

/* syrk */
CLBlastStatusCode CLBlastSsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld,
    const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastCsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset,
    const size_t c_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset,
    const size_t c_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastHsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t
    c_ld, const CUcontext context, const CUdevice device);

/* herk */
CLBlastStatusCode CLBlastCherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset,
    const size_t a_ld, const float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const
    CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld,
    const CUcontext context, const CUdevice device);

/* syr2k */
CLBlastStatusCode CLBlastSsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const float alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const float
    beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice
    device);
CLBlastStatusCode CLBlastDsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const double alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const double
    beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const CUdevice
    device);
CLBlastStatusCode CLBlastCsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexFloat beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context,
    const CUdevice device);
CLBlastStatusCode CLBlastZsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastComplexDouble beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext
    context, const CUdevice device);
CLBlastStatusCode CLBlastHsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t
    a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    CLBlastHalf beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device);

/* her2k */
CLBlastStatusCode CLBlastCher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    float beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastZher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const size_t n, const size_t k, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const
    size_t a_offset, const size_t a_ld, const CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const
    double beta, CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const CUcontext context, const
    CUdevice device);

/* trmm */
CLBlastStatusCode CLBlastStrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const float
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const double
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastCtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const
    CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const
    CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastHtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const
    CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);

/* trsm */
CLBlastStatusCode CLBlastStrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const float
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const double
    alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr b_buffer, const size_t
    b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastCtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const
    CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle,
    const CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const size_t m, const size_t n, const
    CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);

/* omatcopy */
CLBlastStatusCode CLBlastSomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const size_t m,
    const size_t n, const float alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const size_t m,
    const size_t n, const double alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastComatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const size_t m,
    const size_t n, const CLBlastComplexFloat alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t
    a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice
    device);
CLBlastStatusCode CLBlastZomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const size_t m,
    const size_t n, const CLBlastComplexDouble alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t
    a_ld, CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice
    device);
CLBlastStatusCode CLBlastHomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const size_t m,
    const size_t n, const CLBlastHalf alpha, const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld,
    CUdeviceptr b_buffer, const size_t b_offset, const size_t b_ld, const CUcontext context, const CUdevice device);

/* im2col */
CLBlastStatusCode CLBlastSim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastDim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastCim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastZim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastHim2col(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    im_buffer, const size_t im_offset, CUdeviceptr col_buffer, const size_t col_offset, const CUcontext context, const
    CUdevice device);

/* col2im */
CLBlastStatusCode CLBlastScol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastDcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastCcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastZcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastHcol2im(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const CUdeviceptr
    col_buffer, const size_t col_offset, CUdeviceptr im_buffer, const size_t im_offset, const CUcontext context, const
    CUdevice device);

/* convgemm */
CLBlastStatusCode CLBlastSconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device);
CLBlastStatusCode CLBlastDconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device);
CLBlastStatusCode CLBlastHconvgemm(const CLBlastKernelMode kernel_mode, const size_t channels, const size_t height,
    const size_t width, const size_t kernel_h, const size_t kernel_w, const size_t pad_h, const size_t pad_w, const
    size_t stride_h, const size_t stride_w, const size_t dilation_h, const size_t dilation_w, const size_t
    num_kernels, const size_t batch_count, const CUdeviceptr im_buffer, const size_t im_offset, const CUdeviceptr
    kernel_buffer, const size_t kernel_offset, CUdeviceptr result_buffer, const size_t result_offset, const CUcontext
    context, const CUdevice device);

/* gemmBatched */
CLBlastStatusCode CLBlastSgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const float* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const float* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const size_t
    c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastDgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const double* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const double* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const size_t
    c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastCgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexFloat* alphas,
    const CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastComplexFloat* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
    const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexDouble* alphas,
    const CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastComplexDouble* betas, CUdeviceptr c_buffer, const size_t* c_offsets,
    const size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastHgemmBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf* alphas, const
    CUdeviceptr a_buffer, const size_t* a_offsets, const size_t a_ld, const CUdeviceptr b_buffer, const size_t*
    b_offsets, const size_t b_ld, const CLBlastHalf* betas, CUdeviceptr c_buffer, const size_t* c_offsets, const
    size_t c_ld, const size_t batch_count, const CUcontext context, const CUdevice device);

/* gemmStridedBatched */
CLBlastStatusCode CLBlastSgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const float alpha, const CUdeviceptr
    a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const CUdeviceptr b_buffer, const
    size_t b_offset, const size_t b_ld, const size_t b_stride, const float beta, CUdeviceptr c_buffer, const size_t
    c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count, const CUcontext context, const
    CUdevice device);
CLBlastStatusCode CLBlastDgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const double alpha, const
    CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const size_t b_stride, const double beta, CUdeviceptr c_buffer, const
    size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count, const CUcontext context,
    const CUdevice device);
CLBlastStatusCode CLBlastCgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexFloat alpha,
    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const CLBlastComplexFloat beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count,
    const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastZgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastComplexDouble alpha,
    const CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const CUdeviceptr
    b_buffer, const size_t b_offset, const size_t b_ld, const size_t b_stride, const CLBlastComplexDouble beta,
    CUdeviceptr c_buffer, const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count,
    const CUcontext context, const CUdevice device);
CLBlastStatusCode CLBlastHgemmStridedBatched(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const
    CLBlastTranspose b_transpose, const size_t m, const size_t n, const size_t k, const CLBlastHalf alpha, const
    CUdeviceptr a_buffer, const size_t a_offset, const size_t a_ld, const size_t a_stride, const CUdeviceptr b_buffer,
    const size_t b_offset, const size_t b_ld, const size_t b_stride, const CLBlastHalf beta, CUdeviceptr c_buffer,
    const size_t c_offset, const size_t c_ld, const size_t c_stride, const size_t batch_count, const CUcontext
    context, const CUdevice device);

#ifdef __cplusplus
}
#endif

#endif /* B200BLAS_C_H_ */
