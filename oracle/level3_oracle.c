/* CPU oracle for the level-3 routines built on GEMM. TEST INFRASTRUCTURE ONLY.
 *
 * Restates, in plain C and in double precision (complex double for the complex types), what CLBlast's Symm, Hemm,
 * Syrk, Herk, Syr2k, Her2k, Trmm and Trsm compute, so that the CUDA path can be checked against it. Nothing in the
 * product library links, loads or calls it.
 *
 * What is restated, and where the reference defines it:
 *   Symm / Hemm   the stored triangle is mirrored (conjugated, with a real diagonal, for Hemm) into a square matrix,
 *                 then C = alpha*A*B + beta*C (left) or alpha*B*A + beta*C (right): src/routines/level3/xsymm.cpp:33-96,
 *                 xhemm.cpp:33-96, src/kernels/level3/convert_symmetric.opencl, convert_hermitian.opencl;
 *   Syrk / Herk   C = alpha*op(A)*op(A)' + beta*C on one triangle of C, op(A)' the (conjugate) transpose; Herk keeps
 *                 the diagonal real: xsyrk.cpp:51-160, xherk.cpp:51-165, masked write-back
 *                 src/kernels/level3/copy_pad.opencl:84-115;
 *   Syr2k / Her2k two such products, the second with A and B exchanged (and alpha conjugated for Her2k):
 *                 xsyr2k.cpp:33-50, xher2k.cpp:33-52;
 *   Trmm          the triangle is expanded with zeros (ones on a unit diagonal), then B = alpha*op(A)*B or
 *                 alpha*B*op(A): xtrmm.cpp:33-110, src/kernels/level3/convert_triangular.opencl;
 *   Trsm          the X with op(A)*X = alpha*B or X*op(A) = alpha*B. The reference obtains it from inverted diagonal
 *                 blocks and GEMM updates (xtrsm.cpp:40-243); the oracle uses plain substitution, the definition both
 *                 approximate.
 * Parity pin: the reference's own tests compare these routines with a CBLAS library on seeded data and hold no golden
 * vectors (test/routines/level3/xsymm.hpp:113-121 and siblings). The square-matrix expansions are pinned against the
 * reference's convert kernels run on the CPU (oracle/build_ref.py, tests/test_oracle_ref.py); the products go through
 * the GEMM arithmetic that is pinned the same way; the routines as a whole are checked against independent numpy
 * evaluations of the BLAS definitions (tests/test_oracle.py).
 *
 * Inputs are typed buffers (dtype 16, 32, 64, 3232, 6464 as in gemm_oracle.c); the matrix that is written is a
 * double buffer of the same geometry (pairs for the complex types), updated in place. */
#include <complex.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ROW_MAJOR 101
#define TR_NO 111
#define TR_CONJ 113
#define TRI_UPPER 121
#define DIAG_UNIT 132
#define SIDE_LEFT 141

typedef double complex zc;
typedef _Float16 f16;

static int is_complex(int dtype) { return dtype == 3232 || dtype == 6464; }

static zc load(int dtype, const void* p, size_t i) {
  switch (dtype) {
    case 16: { f16 v; memcpy(&v, (const uint16_t*)p + i, 2); return (double)v; }
    case 32: return ((const float*)p)[i];
    case 64: return ((const double*)p)[i];
    case 3232: return ((const float*)p)[2 * i] + I * ((const float*)p)[2 * i + 1];
    default: return ((const double*)p)[2 * i] + I * ((const double*)p)[2 * i + 1];
  }
}

static size_t at(int layout, size_t r, size_t c, size_t ld) { return layout == ROW_MAJOR ? r * ld + c : c * ld + r; }

static zc wide_get(int cplx, const double* w, size_t i) { return cplx ? w[2 * i] + I * w[2 * i + 1] : w[i]; }
static void wide_set(int cplx, double* w, size_t i, zc v) {
  if (cplx) { w[2 * i] = creal(v); w[2 * i + 1] = cimag(v); } else { w[i] = creal(v); }
}

/* rows x cols, row-major: op(X) of a general typed matrix. */
static zc* dense_general(int dtype, int layout, int trans, size_t rows, size_t cols, const void* x, size_t off, size_t ld) {
  zc* d = (zc*)malloc(sizeof(zc) * rows * cols);
  if (!d) return NULL;
  for (size_t r = 0; r < rows; ++r)
    for (size_t c = 0; c < cols; ++c) {
      zc v = (trans == TR_NO) ? load(dtype, x, off + at(layout, r, c, ld)) : load(dtype, x, off + at(layout, c, r, ld));
      d[r * cols + c] = (trans == TR_CONJ) ? conj(v) : v;
    }
  return d;
}

/* k x k, row-major, from the stored triangle. kind 0 symmetric, 1 hermitian, 2 triangular. */
static zc* dense_from_triangle(int dtype, int kind, int layout, int triangle, int unit, size_t k, const void* a, size_t off,
                               size_t ld) {
  zc* d = (zc*)malloc(sizeof(zc) * k * k);
  if (!d) return NULL;
  for (size_t r = 0; r < k; ++r)
    for (size_t c = 0; c < k; ++c) {
      const int stored = (triangle == TRI_UPPER) ? (r <= c) : (r >= c);
      zc v;
      if (stored) {
        v = load(dtype, a, off + at(layout, r, c, ld));
        if (kind == 1 && r == c) v = creal(v);
        if (kind == 2 && r == c && unit) v = 1.0;
      } else if (kind == 2) {
        v = 0.0;
      } else {
        v = load(dtype, a, off + at(layout, c, r, ld));
        if (kind == 1) v = conj(v);
      }
      d[r * k + c] = v;
    }
  return d;
}

/* The expanded square matrix itself, as a double buffer in MEMORY order (element (r, c) of the k x k result at
 * c*k + r when column-major, r*k + c when row-major): what the reference's convert kernels produce. */
int oracle_expand_triangle(int dtype, int kind, int layout, int triangle, int unit, size_t k, const void* a, size_t a_off,
                           size_t a_ld, double* out) {
  zc* d = dense_from_triangle(dtype, kind, layout, triangle, unit, k, a, a_off, a_ld);
  if (!d) return -1;
  const int cplx = is_complex(dtype);
  for (size_t r = 0; r < k; ++r)
    for (size_t c = 0; c < k; ++c) wide_set(cplx, out, at(layout, r, c, k), d[r * k + c]);
  free(d);
  return 0;
}

int oracle_symm_f64(int dtype, int hermitian, int layout, int side, int triangle, size_t m, size_t n, const double* alpha,
                    const void* a, size_t a_off, size_t a_ld, const void* b, size_t b_off, size_t b_ld,
                    const double* beta, double* c64, size_t c_off, size_t c_ld) {
  const int cplx = is_complex(dtype);
  const size_t k = (side == SIDE_LEFT) ? m : n;
  zc* sq = dense_from_triangle(dtype, hermitian ? 1 : 0, layout, triangle, 0, k, a, a_off, a_ld);
  zc* bd = dense_general(dtype, layout, TR_NO, m, n, b, b_off, b_ld);
  if (!sq || !bd) return -1;
  const zc al = alpha[0] + I * alpha[1], be = beta[0] + I * beta[1];
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      zc acc = 0.0;
      if (side == SIDE_LEFT) for (size_t l = 0; l < k; ++l) acc += sq[i * k + l] * bd[l * n + j];
      else for (size_t l = 0; l < k; ++l) acc += bd[i * n + l] * sq[l * k + j];
      const size_t ci = c_off + at(layout, i, j, c_ld);
      const zc old = (be == 0.0) ? 0.0 : be * wide_get(cplx, c64, ci);
      wide_set(cplx, c64, ci, al * acc + old);
    }
  free(sq); free(bd);
  return 0;
}

/* One masked product C(triangle) = alpha*op(A)*op(B)' + beta*C; op is `trans`, ' the (conjugate) transpose. */
static int rank_k(int dtype, int hermitian, int layout, int triangle, int trans, size_t n, size_t k, zc al, const void* a,
                  size_t a_off, size_t a_ld, const void* b, size_t b_off, size_t b_ld, zc be, double* c64, size_t c_off,
                  size_t c_ld, int real_diag) {
  const int cplx = is_complex(dtype);
  const int t = (trans == TR_NO) ? TR_NO : (hermitian ? TR_CONJ : 112);
  zc* ad = dense_general(dtype, layout, t, n, k, a, a_off, a_ld);   /* op(A): n x k */
  zc* bd = dense_general(dtype, layout, t, n, k, b, b_off, b_ld);   /* op(B): n x k */
  if (!ad || !bd) return -1;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i)
    for (size_t j = 0; j < n; ++j) {
      if ((triangle == TRI_UPPER) ? (i > j) : (i < j)) continue;
      zc acc = 0.0;
      for (size_t l = 0; l < k; ++l) acc += ad[i * k + l] * (hermitian ? conj(bd[j * k + l]) : bd[j * k + l]);
      const size_t ci = c_off + at(layout, i, j, c_ld);
      zc v = al * acc + ((be == 0.0) ? 0.0 : be * wide_get(cplx, c64, ci));
      if (real_diag && i == j) v = creal(v);
      wide_set(cplx, c64, ci, v);
    }
  free(ad); free(bd);
  return 0;
}

int oracle_syrk_f64(int dtype, int hermitian, int layout, int triangle, int trans, size_t n, size_t k, const double* alpha,
                    const void* a, size_t a_off, size_t a_ld, const double* beta, double* c64, size_t c_off, size_t c_ld) {
  return rank_k(dtype, hermitian, layout, triangle, trans, n, k, alpha[0] + I * alpha[1], a, a_off, a_ld, a, a_off, a_ld,
                beta[0] + I * beta[1], c64, c_off, c_ld, hermitian);
}

int oracle_syr2k_f64(int dtype, int hermitian, int layout, int triangle, int trans, size_t n, size_t k,
                     const double* alpha, const void* a, size_t a_off, size_t a_ld, const void* b, size_t b_off,
                     size_t b_ld, const double* beta, double* c64, size_t c_off, size_t c_ld) {
  const zc al = alpha[0] + I * alpha[1];
  int st = rank_k(dtype, hermitian, layout, triangle, trans, n, k, al, a, a_off, a_ld, b, b_off, b_ld,
                  beta[0] + I * beta[1], c64, c_off, c_ld, 0);
  if (st) return st;
  return rank_k(dtype, hermitian, layout, triangle, trans, n, k, hermitian ? conj(al) : al, b, b_off, b_ld, a, a_off, a_ld,
                1.0, c64, c_off, c_ld, hermitian);
}

/* op(A) as a dense k x k row-major matrix of the triangular A. */
static zc* dense_op_triangular(int dtype, int layout, int triangle, int trans, int diag, size_t k, const void* a,
                               size_t a_off, size_t a_ld) {
  zc* t = dense_from_triangle(dtype, 2, layout, triangle, diag == DIAG_UNIT, k, a, a_off, a_ld);
  if (!t || trans == TR_NO) return t;
  zc* o = (zc*)malloc(sizeof(zc) * k * k);
  if (!o) { free(t); return NULL; }
  for (size_t r = 0; r < k; ++r)
    for (size_t c = 0; c < k; ++c) o[r * k + c] = (trans == TR_CONJ) ? conj(t[c * k + r]) : t[c * k + r];
  free(t);
  return o;
}

int oracle_trmm_f64(int dtype, int layout, int side, int triangle, int trans, int diag, size_t m, size_t n,
                    const double* alpha, const void* a, size_t a_off, size_t a_ld, double* b64, size_t b_off, size_t b_ld) {
  const int cplx = is_complex(dtype);
  const size_t k = (side == SIDE_LEFT) ? m : n;
  zc* t = dense_op_triangular(dtype, layout, triangle, trans, diag, k, a, a_off, a_ld);
  zc* bd = (zc*)malloc(sizeof(zc) * m * n);
  if (!t || !bd) return -1;
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) bd[i * n + j] = wide_get(cplx, b64, b_off + at(layout, i, j, b_ld));
  const zc al = alpha[0] + I * alpha[1];
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) {
      zc acc = 0.0;
      if (side == SIDE_LEFT) for (size_t l = 0; l < k; ++l) acc += t[i * k + l] * bd[l * n + j];
      else for (size_t l = 0; l < k; ++l) acc += bd[i * n + l] * t[l * k + j];
      wide_set(cplx, b64, b_off + at(layout, i, j, b_ld), al * acc);
    }
  free(t); free(bd);
  return 0;
}

int oracle_trsm_f64(int dtype, int layout, int side, int triangle, int trans, int diag, size_t m, size_t n,
                    const double* alpha, const void* a, size_t a_off, size_t a_ld, double* b64, size_t b_off, size_t b_ld) {
  const int cplx = is_complex(dtype);
  const size_t k = (side == SIDE_LEFT) ? m : n;
  zc* t = dense_op_triangular(dtype, layout, triangle, trans, diag, k, a, a_off, a_ld);   /* op(A), k x k */
  zc* x = (zc*)malloc(sizeof(zc) * m * n);
  if (!t || !x) return -1;
  const zc al = alpha[0] + I * alpha[1];
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) x[i * n + j] = al * wide_get(cplx, b64, b_off + at(layout, i, j, b_ld));
  const int op_lower = (triangle == TRI_UPPER) != (trans == TR_NO);
  if (side == SIDE_LEFT) {        /* op(A) X = alpha B, column by column */
#pragma omp parallel for schedule(static)
    for (size_t j = 0; j < n; ++j) {
      for (size_t s = 0; s < k; ++s) {
        const size_t i = op_lower ? s : k - 1 - s;
        zc acc = x[i * n + j];
        if (op_lower) for (size_t l = 0; l < i; ++l) acc -= t[i * k + l] * x[l * n + j];
        else for (size_t l = i + 1; l < k; ++l) acc -= t[i * k + l] * x[l * n + j];
        x[i * n + j] = acc / t[i * k + i];
      }
    }
  } else {                        /* X op(A) = alpha B, row by row */
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < m; ++i) {
      for (size_t s = 0; s < k; ++s) {
        const size_t j = op_lower ? k - 1 - s : s;
        zc acc = x[i * n + j];
        if (op_lower) for (size_t l = j + 1; l < k; ++l) acc -= x[i * n + l] * t[l * k + j];
        else for (size_t l = 0; l < j; ++l) acc -= x[i * n + l] * t[l * k + j];
        x[i * n + j] = acc / t[j * k + j];
      }
    }
  }
  for (size_t i = 0; i < m; ++i)
    for (size_t j = 0; j < n; ++j) wide_set(cplx, b64, b_off + at(layout, i, j, b_ld), x[i * n + j]);
  free(t); free(x);
  return 0;
}
