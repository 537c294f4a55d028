/* Host-pointer BLAS interface over libclblast.so, with the names and argument lists of the reference's Netlib layer
 * (include/clblast_netlib_c.h:402-519; implementation src/clblast_netlib_c.cpp:2718-2749 and following): matrices are
 * HOST arrays. Every call copies its operands to the current CUDA device, runs the device routine and copies the
 * result back, so it is a convenience layer, not a fast path. As in the reference, a failing call throws
 * std::runtime_error("CLBlast returned with error code <n>") through the C interface. Complex scalars are passed by
 * pointer to (re, im). */
#ifndef B200BLAS_NETLIB_H_
#define B200BLAS_NETLIB_H_

#include "b200blas_c.h"

#ifdef __cplusplus
extern "C" {
#endif


/* gemm */
void cblas_sgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose b_transpose,
    const int m, const int n, const int k, const float alpha, const float* a, const int a_ld, const float* b, const
    int b_ld, const float beta, float* c, const int c_ld);
void cblas_dgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose b_transpose,
    const int m, const int n, const int k, const double alpha, const double* a, const int a_ld, const double* b, const
    int b_ld, const double beta, double* c, const int c_ld);
void cblas_cgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose b_transpose,
    const int m, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const void* beta, void* c, const int c_ld);
void cblas_zgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose b_transpose,
    const int m, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const void* beta, void* c, const int c_ld);

/* symm */
void cblas_ssymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const float alpha, const float* a, const int a_ld, const float* b, const int b_ld, const float beta,
    float* c, const int c_ld);
void cblas_dsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const double alpha, const double* a, const int a_ld, const double* b, const int b_ld, const double
    beta, double* c, const int c_ld);
void cblas_csymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void* beta,
    void* c, const int c_ld);
void cblas_zsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void* beta,
    void* c, const int c_ld);

/* hemm */
void cblas_chemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void* beta,
    void* c, const int c_ld);
void cblas_zhemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const int m,
    const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void* beta,
    void* c, const int c_ld);

/* syrk */
void cblas_ssyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const float alpha, const float* a, const int a_ld, const float beta, float* c, const int
    c_ld);
void cblas_dsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const double alpha, const double* a, const int a_ld, const double beta, double* c, const int
    c_ld);
void cblas_csyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const void* alpha, const void* a, const int a_ld, const void* beta, void* c, const int c_ld);
void cblas_zsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const void* alpha, const void* a, const int a_ld, const void* beta, void* c, const int c_ld);

/* herk */
void cblas_cherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const float alpha, const void* a, const int a_ld, const float beta, void* c, const int c_ld);
void cblas_zherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose a_transpose, const
    int n, const int k, const double alpha, const void* a, const int a_ld, const double beta, void* c, const int
    c_ld);

/* syr2k */
void cblas_ssyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const float alpha, const float* a, const int a_ld, const float* b, const int b_ld, const
    float beta, float* c, const int c_ld);
void cblas_dsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const double alpha, const double* a, const int a_ld, const double* b, const int b_ld,
    const double beta, double* c, const int c_ld);
void cblas_csyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const
    void* beta, void* c, const int c_ld);
void cblas_zsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const
    void* beta, void* c, const int c_ld);

/* her2k */
void cblas_cher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const
    float beta, void* c, const int c_ld);
void cblas_zher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose ab_transpose,
    const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const
    double beta, void* c, const int c_ld);

/* trmm */
void cblas_strmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const float alpha, const
    float* a, const int a_ld, float* b, const int b_ld);
void cblas_dtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const double alpha, const
    double* a, const int a_ld, double* b, const int b_ld);
void cblas_ctrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld);
void cblas_ztrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld);

/* trsm */
void cblas_strsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const float alpha, const
    float* a, const int a_ld, float* b, const int b_ld);
void cblas_dtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const double alpha, const
    double* a, const int a_ld, double* b, const int b_ld);
void cblas_ctrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld);
void cblas_ztrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld);

/* omatcopy */
void cblas_somatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int n, const
    float alpha, const float* a, const int a_ld, float* b, const int b_ld);
void cblas_domatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int n, const
    double alpha, const double* a, const int a_ld, double* b, const int b_ld);
void cblas_comatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int n, const
    void* alpha, const void* a, const int a_ld, void* b, const int b_ld);
void cblas_zomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int n, const
    void* alpha, const void* a, const int a_ld, void* b, const int b_ld);

#ifdef __cplusplus
}
#endif

#endif /* B200BLAS_NETLIB_H_ */
