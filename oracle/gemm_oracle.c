/* CPU oracle for the GEMM hot path. TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of CLBlast's GEMM family so that the CUDA kernels can be
 * checked against it. Nothing in the product library links, loads or calls it; only tests/, the smoke check
 * and the CPU-baseline leg of bench.py do.
 *
 * Parity pin: the reference ships no golden vectors or known-answer files for this path; its tests compare
 * two implementations on seeded random data. This oracle is pinned instead (a) against the reference's own
 * kernel source, compiled for the CPU by oracle/build_ref.py into oracle/_ref/ and executed work-group by
 * work-group (tests/test_oracle_ref.py: bit-identical for half, single and double), and (b) against fixtures under tests/golden/ generated with numpy's
 * fp64 product.
 *
 * Two flavours of every routine:
 *   oracle_*        "reference order": per output element acc = 0; for k ascending: acc += a*b; then
 *                   alpha*acc (+ beta*c when beta != 0), all in the routine's own type T. This is what the
 *                   reference kernels compute (src/kernels/level3/xgemm_direct_part3.opencl:41-135,
 *                   src/kernels/level3/xgemm_part3.opencl:98-304, AXPBY and MultiplyAdd in
 *                   src/kernels/common.opencl:208-244). T = half accumulates in half, as the reference does.
 *   oracle_*_f64    the same sums with every input widened to double: the accuracy yardstick.
 * Addressing follows the reference's API: element (i,j) of a matrix with leading dimension ld sits at
 * offset + (row-major ? i*ld + j : j*ld + i), with the transpose flags swapping the roles of i and j
 * (test/routines/level3/xgemm.hpp:174-177, src/routines/level3/xgemm.hpp:87-107).
 *
 * dtype codes: 16 half (uint16 bit patterns), 32 float, 64 double, 3232 complex float, 6464 complex double.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ROW_MAJOR 101
#define COL_MAJOR 102
#define TR_NO 111
#define TR_YES 112
#define TR_CONJ 113
#define MODE_CONVOLUTION 152

typedef _Float16 f16;

static inline double half_to_double(uint16_t h) {
  f16 v;
  memcpy(&v, &h, 2);
  return (double)v;
}

/* Index of op(X)(r, c) in storage, where `trans` says op transposes the stored matrix. */
static inline size_t idx(int layout, int trans, size_t r, size_t c, size_t ld) {
  const int stored_row_is_r = (trans == TR_NO);
  const size_t sr = stored_row_is_r ? r : c;
  const size_t sc = stored_row_is_r ? c : r;
  return (layout == ROW_MAJOR) ? sr * ld + sc : sc * ld + sr;
}

/* Loads element `i` of a typed buffer as (re, im) doubles. */
static inline void load2(int dtype, const void* p, size_t i, double* re, double* im) {
  *im = 0.0;
  switch (dtype) {
    case 16: *re = half_to_double(((const uint16_t*)p)[i]); break;
    case 32: *re = ((const float*)p)[i]; break;
    case 64: *re = ((const double*)p)[i]; break;
    case 3232: *re = ((const float*)p)[2 * i]; *im = ((const float*)p)[2 * i + 1]; break;
    default: *re = ((const double*)p)[2 * i]; *im = ((const double*)p)[2 * i + 1]; break;
  }
}

static int is_complex(int dtype) { return dtype == 3232 || dtype == 6464; }

/* Packs op(A) (rows x cols, row-major, compute type double pairs) out of the typed source. */
static void pack_f64(int dtype, int layout, int trans, size_t rows, size_t cols, const void* src, size_t off,
                     size_t ld, double* re, double* im) {
#pragma omp parallel for schedule(static)
  for (size_t r = 0; r < rows; ++r) {
    for (size_t c = 0; c < cols; ++c) {
      double x, y;
      load2(dtype, src, off + idx(layout, trans, r, c, ld), &x, &y);
      if (trans == TR_CONJ) y = -y;
      re[r * cols + c] = x;
      if (im) im[r * cols + c] = y;
    }
  }
}

/* ---- fp64 yardstick ---------------------------------------------------------------------------------- */

/* c64 holds the C buffer widened to double (pairs for complex), same geometry as the typed C buffer
 * (c_offset, c_ld, layout); it is updated in place: C = alpha*op(A)*op(B) + beta*C, beta == 0 ignoring C. */
int oracle_gemm_f64(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const double* alpha,
                    const void* a, size_t a_off, size_t a_ld, const void* b, size_t b_off, size_t b_ld,
                    const double* beta, double* c64, size_t c_off, size_t c_ld) {
  const int cplx = is_complex(dtype);
  double* are = (double*)malloc(sizeof(double) * m * k);
  double* bre = (double*)malloc(sizeof(double) * k * n);
  double* aim = cplx ? (double*)malloc(sizeof(double) * m * k) : NULL;
  double* bim = cplx ? (double*)malloc(sizeof(double) * k * n) : NULL;
  if (!are || !bre || (cplx && (!aim || !bim))) return -1;
  pack_f64(dtype, layout, ta, m, k, a, a_off, a_ld, are, aim);
  pack_f64(dtype, layout, tb, k, n, b, b_off, b_ld, bre, bim);
  const int use_beta = !(beta[0] == 0.0 && (!cplx || beta[1] == 0.0));
#pragma omp parallel
  {
    double* accr = (double*)malloc(sizeof(double) * n);
    double* acci = cplx ? (double*)malloc(sizeof(double) * n) : NULL;
#pragma omp for schedule(dynamic, 4)
    for (size_t i = 0; i < m; ++i) {
      for (size_t j = 0; j < n; ++j) accr[j] = 0.0;
      if (cplx) for (size_t j = 0; j < n; ++j) acci[j] = 0.0;
      for (size_t l = 0; l < k; ++l) {
        const double ar = are[i * k + l];
        const double* br = bre + l * n;
        if (!cplx) {
          for (size_t j = 0; j < n; ++j) accr[j] += ar * br[j];
        } else {
          const double ai = aim[i * k + l];
          const double* bi = bim + l * n;
          for (size_t j = 0; j < n; ++j) {
            accr[j] += ar * br[j] - ai * bi[j];
            acci[j] += ar * bi[j] + ai * br[j];
          }
        }
      }
      for (size_t j = 0; j < n; ++j) {
        const size_t ci = c_off + ((layout == ROW_MAJOR) ? i * c_ld + j : j * c_ld + i);
        if (!cplx) {
          c64[ci] = use_beta ? alpha[0] * accr[j] + beta[0] * c64[ci] : alpha[0] * accr[j];
        } else {
          double rr = alpha[0] * accr[j] - alpha[1] * acci[j];
          double ri = alpha[0] * acci[j] + alpha[1] * accr[j];
          if (use_beta) {
            const double cr = c64[2 * ci], cim = c64[2 * ci + 1];
            rr += beta[0] * cr - beta[1] * cim;
            ri += beta[0] * cim + beta[1] * cr;
          }
          c64[2 * ci] = rr;
          c64[2 * ci + 1] = ri;
        }
      }
    }
    free(accr);
    free(acci);
  }
  free(are); free(bre); free(aim); free(bim);
  return 0;
}

/* Exact fp64 values alpha*sum_k op(A)(i,k) op(B)(k,j) (no beta term) for `count` sampled (rows[s], cols[s]);
 * real dtypes only. Also returns sum_k |a||b| per sample for normalised error reporting. */
int oracle_gemm_f64_sampled(int dtype, int layout, int ta, int tb, size_t k, double alpha, const void* a, size_t a_off,
                            size_t a_ld, const void* b, size_t b_off, size_t b_ld, size_t count, const size_t* rows,
                            const size_t* cols, double* out, double* out_abs) {
  if (is_complex(dtype)) return -1;
#pragma omp parallel for schedule(dynamic, 16)
  for (size_t s = 0; s < count; ++s) {
    double acc = 0.0, mag = 0.0;
    for (size_t l = 0; l < k; ++l) {
      double x, y, u;
      load2(dtype, a, a_off + idx(layout, ta, rows[s], l, a_ld), &x, &u);
      load2(dtype, b, b_off + idx(layout, tb, l, cols[s], b_ld), &y, &u);
      acc += x * y;
      mag += fabs(x * y);
    }
    out[s] = alpha * acc;
    if (out_abs) out_abs[s] = mag;
  }
  return 0;
}

/* ---- reference-order, type-T ------------------------------------------------------------------------- */

#define DEFINE_REAL_GEMM(NAME, T, FMA, AXPBY)                                                                         \
  static int NAME(int layout, int ta, int tb, size_t m, size_t n, size_t k, T alpha, const T* a, size_t a_off, \
                  size_t a_ld, const T* b, size_t b_off, size_t b_ld, T beta, T* c, size_t c_off, size_t c_ld) { \
    T* ap = (T*)malloc(sizeof(T) * m * k);                                                                     \
    T* bp = (T*)malloc(sizeof(T) * k * n);                                                                     \
    if (!ap || !bp) return -1;                                                                                 \
    _Pragma("omp parallel for schedule(static)") for (size_t i = 0; i < m; ++i) for (size_t l = 0; l < k; ++l) \
        ap[i * k + l] = a[a_off + idx(layout, ta, i, l, a_ld)];                                                \
    _Pragma("omp parallel for schedule(static)") for (size_t l = 0; l < k; ++l) for (size_t j = 0; j < n; ++j) \
        bp[l * n + j] = b[b_off + idx(layout, tb, l, j, b_ld)];                                                \
    _Pragma("omp parallel") {                                                                                  \
      T* acc = (T*)malloc(sizeof(T) * n);                                                                      \
      _Pragma("omp for schedule(dynamic, 4)") for (size_t i = 0; i < m; ++i) {                                 \
        for (size_t j = 0; j < n; ++j) acc[j] = (T)0;                                                          \
        for (size_t l = 0; l < k; ++l) {                                                                       \
          const T av = ap[i * k + l];                                                                          \
          const T* br = bp + l * n;                                                                            \
          for (size_t j = 0; j < n; ++j) acc[j] = FMA(av, br[j], acc[j]);                                      \
        }                                                                                                      \
        for (size_t j = 0; j < n; ++j) {                                                                       \
          const size_t ci = c_off + ((layout == ROW_MAJOR) ? i * c_ld + j : j * c_ld + i);                     \
          /* alpha*acc + beta*c evaluated as fma(beta, c, alpha*acc): the contraction the reference's AXPBY     \
           * (src/kernels/common.opencl:240-244) gets from a fusing compiler; bit-identical to the reference's  \
           * kernel source executed on the CPU (tests/test_oracle_ref.py). */                                  \
          c[ci] = (beta == (T)0) ? (T)(alpha * acc[j]) : (T)(AXPBY(alpha, acc[j], beta, c[ci]));                            \
        }                                                                                                      \
      }                                                                                                        \
      free(acc);                                                                                               \
    }                                                                                                          \
    free(ap); free(bp);                                                                                        \
    return 0;                                                                                                  \
  }

#define FMA_F32(a, b, c) fmaf((a), (b), (c))
#define FMA_F64(a, b, c) fma((a), (b), (c))
/* Half: the product of two halves is exact in float; the sum is formed in float and rounded to half, which is
 * what `acc += a*b` on half operands gives on a target that evaluates half arithmetic in float. */
#define FMA_F16(a, b, c) ((f16)((float)(a) * (float)(b) + (float)(c)))

#define AXPBY_F32(al, x, be, y) fmaf((be), (y), (al) * (x))
#define AXPBY_F64(al, x, be, y) fma((be), (y), (al) * (x))
/* Half: both products are exact in float, one float addition, one rounding to half. */
#define AXPBY_F16(al, x, be, y) ((f16)((float)(al) * (float)(x) + (float)(be) * (float)(y)))

DEFINE_REAL_GEMM(gemm_f32, float, FMA_F32, AXPBY_F32)
DEFINE_REAL_GEMM(gemm_f64, double, FMA_F64, AXPBY_F64)
DEFINE_REAL_GEMM(gemm_f16, f16, FMA_F16, AXPBY_F16)

#define DEFINE_COMPLEX_GEMM(NAME, R)                                                                           \
  static int NAME(int layout, int ta, int tb, size_t m, size_t n, size_t k, const R* alpha, const R* a,        \
                  size_t a_off, size_t a_ld, const R* b, size_t b_off, size_t b_ld, const R* beta, R* c,       \
                  size_t c_off, size_t c_ld) {                                                                 \
    const int use_beta = !(beta[0] == (R)0 && beta[1] == (R)0);                                                \
    _Pragma("omp parallel for schedule(dynamic, 4)") for (size_t i = 0; i < m; ++i) {                          \
      for (size_t j = 0; j < n; ++j) {                                                                         \
        R accr = 0, acci = 0;                                                                                  \
        for (size_t l = 0; l < k; ++l) {                                                                       \
          const size_t ai = a_off + idx(layout, ta, i, l, a_ld);                                               \
          const size_t bi = b_off + idx(layout, tb, l, j, b_ld);                                               \
          const R ar = a[2 * ai], aim = (ta == TR_CONJ) ? -a[2 * ai + 1] : a[2 * ai + 1];                      \
          const R br = b[2 * bi], bim = (tb == TR_CONJ) ? -b[2 * bi + 1] : b[2 * bi + 1];                      \
          accr += ar * br - aim * bim;                                                                         \
          acci += ar * bim + aim * br;                                                                         \
        }                                                                                                      \
        const size_t ci = c_off + ((layout == ROW_MAJOR) ? i * c_ld + j : j * c_ld + i);                       \
        R rr = alpha[0] * accr - alpha[1] * acci;                                                              \
        R ri = alpha[0] * acci + alpha[1] * accr;                                                              \
        if (use_beta) {                                                                                        \
          const R cr = c[2 * ci], cim = c[2 * ci + 1];                                                         \
          rr += beta[0] * cr - beta[1] * cim;                                                                  \
          ri += beta[0] * cim + beta[1] * cr;                                                                  \
        }                                                                                                      \
        c[2 * ci] = rr;                                                                                        \
        c[2 * ci + 1] = ri;                                                                                    \
      }                                                                                                        \
    }                                                                                                          \
    return 0;                                                                                                  \
  }

DEFINE_COMPLEX_GEMM(gemm_c32, float)
DEFINE_COMPLEX_GEMM(gemm_c64, double)

/* In-place on the host C buffer, exactly like the API: alpha and beta point to one scalar of the dtype. */
int oracle_gemm(int dtype, int layout, int ta, int tb, size_t m, size_t n, size_t k, const void* alpha, const void* a,
                size_t a_off, size_t a_ld, const void* b, size_t b_off, size_t b_ld, const void* beta, void* c,
                size_t c_off, size_t c_ld) {
  switch (dtype) {
    case 32:
      return gemm_f32(layout, ta, tb, m, n, k, *(const float*)alpha, (const float*)a, a_off, a_ld, (const float*)b,
                      b_off, b_ld, *(const float*)beta, (float*)c, c_off, c_ld);
    case 64:
      return gemm_f64(layout, ta, tb, m, n, k, *(const double*)alpha, (const double*)a, a_off, a_ld, (const double*)b,
                      b_off, b_ld, *(const double*)beta, (double*)c, c_off, c_ld);
    case 16: {
      f16 al, be;
      memcpy(&al, alpha, 2);
      memcpy(&be, beta, 2);
      return gemm_f16(layout, ta, tb, m, n, k, al, (const f16*)a, a_off, a_ld, (const f16*)b, b_off, b_ld, be,
                      (f16*)c, c_off, c_ld);
    }
    case 3232:
      return gemm_c32(layout, ta, tb, m, n, k, (const float*)alpha, (const float*)a, a_off, a_ld, (const float*)b,
                      b_off, b_ld, (const float*)beta, (float*)c, c_off, c_ld);
    case 6464:
      return gemm_c64(layout, ta, tb, m, n, k, (const double*)alpha, (const double*)a, a_off, a_ld, (const double*)b,
                      b_off, b_ld, (const double*)beta, (double*)c, c_off, c_ld);
    default: return -2;
  }
}

/* ---- convolution -------------------------------------------------------------------------------------- */

/* Output extents as computed by the routine (src/routines/levelx/xconvgemm.cpp:67-72). */
void oracle_conv_output_size(size_t height, size_t width, size_t kernel_h, size_t kernel_w, size_t pad_h, size_t pad_w,
                             size_t stride_h, size_t stride_w, size_t dil_h, size_t dil_w, size_t* out_h,
                             size_t* out_w) {
  const size_t size_h = height + 2 * pad_h, padding_h = dil_h * (kernel_h - 1) + 1;
  const size_t size_w = width + 2 * pad_w, padding_w = dil_w * (kernel_w - 1) + 1;
  *out_h = (size_h >= padding_h) ? (size_h - padding_h) / stride_h + 1 : 1;
  *out_w = (size_w >= padding_w) ? (size_w - padding_w) / stride_w + 1 : 1;
}

/* Direct convolution with the summation order of the reference KERNEL (src/kernels/levelx/xconvgemm_part1.opencl:
 * 31-53, xconvgemm_part2.opencl:27-285): for each output pixel and output channel, k = (channel, kh, kw) runs
 * ascending over the WEIGHT index and the image tap is taken at (kh, kw), mirrored to (KH-1-kh, KW-1-kw) for
 * kConvolution; taps outside the image contribute zero. (The reference's host-side test loop,
 * test/routines/levelx/xconvgemm.hpp:151-196, forms the same sum with the weight index mirrored instead.)
 * `result64` (double) is written when non-null, else `result` in the dtype with accumulation in the dtype.
 * Real dtypes only. */
int oracle_convgemm(int dtype, int mode, size_t channels, size_t height, size_t width, size_t kernel_h, size_t kernel_w,
                    size_t pad_h, size_t pad_w, size_t stride_h, size_t stride_w, size_t dil_h, size_t dil_w,
                    size_t num_kernels, size_t batch_count, const void* im, size_t im_off, const void* ker,
                    size_t ker_off, void* result, size_t result_off, double* result64) {
  if (is_complex(dtype)) return -2;
  size_t out_h, out_w;
  oracle_conv_output_size(height, width, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, &out_h,
                          &out_w);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (size_t nb = 0; nb < batch_count; ++nb) {
    for (size_t co = 0; co < num_kernels; ++co) {
      for (size_t ho = 0; ho < out_h; ++ho) {
        for (size_t wo = 0; wo < out_w; ++wo) {
          double acc64 = 0.0;
          float acc32 = 0.f;
          f16 acc16 = (f16)0;
          for (size_t ci = 0; ci < channels; ++ci) {
            for (size_t kh = 0; kh < kernel_h; ++kh) {
              for (size_t kw = 0; kw < kernel_w; ++kw) {
                const size_t th = (mode == MODE_CONVOLUTION) ? kernel_h - kh - 1 : kh;
                const size_t tw = (mode == MODE_CONVOLUTION) ? kernel_w - kw - 1 : kw;
                const long long hi = (long long)(th * dil_h + stride_h * ho) - (long long)pad_h;
                const long long wi = (long long)(tw * dil_w + stride_w * wo) - (long long)pad_w;
                if (hi < 0 || hi >= (long long)height || wi < 0 || wi >= (long long)width) continue;
                const size_t ii = (size_t)wi + width * ((size_t)hi + height * (ci + channels * nb)) + im_off;
                const size_t ki = kw + kernel_w * (kh + kernel_h * (ci + channels * co));
                double x, y, u;
                load2(dtype, im, ii, &x, &u);
                load2(dtype, ker, ki + ker_off, &y, &u);
                if (result64 || dtype == 64) {
                  acc64 = result64 ? acc64 + x * y : fma(x, y, acc64);
                } else if (dtype == 32) {
                  acc32 = fmaf((float)x, (float)y, acc32);
                } else {
                  acc16 = FMA_F16((f16)x, (f16)y, acc16);
                }
              }
            }
          }
          const size_t oi = wo + out_w * (ho + out_h * (co + num_kernels * nb)) + result_off;
          if (result64) {
            result64[oi] = acc64;
          } else if (dtype == 64) {
            ((double*)result)[oi] = acc64;
          } else if (dtype == 32) {
            ((float*)result)[oi] = acc32;
          } else {
            memcpy((uint16_t*)result + oi, &acc16, 2);
          }
        }
      }
    }
  }
  return 0;
}

/* ---- comparison rule ----------------------------------------------------------------------------------- */

/* The reference's pass criterion for one pair of values (test/correctness/tester.cpp:561-593): equal, or both
 * non-finite, or |d| < abs margin when either value is 0 or d is tiny, else |d|/(|x|+|y|) < rel margin. */
static int similar(double x, double y, double abs_margin, double rel_margin) {
  const double d = fabs(x - y);
  if (x == y) return 1;
  if ((isnan(x) || isinf(x)) && (isnan(y) || isinf(y))) return 1;
  if (x == 0.0 || y == 0.0 || d < abs_margin) return d < abs_margin;
  return d / (fabs(x) + fabs(y)) < rel_margin;
}

/* Counts the failures of the rule over `count` pairs; stores the largest |x-y| in *max_abs. */
size_t oracle_count_mismatches(const double* x, const double* y, size_t count, double abs_margin, double rel_margin,
                               double* max_abs) {
  size_t bad = 0;
  double worst = 0.0;
  for (size_t i = 0; i < count; ++i) {
    if (!similar(x[i], y[i], abs_margin, rel_margin)) ++bad;
    const double d = fabs(x[i] - y[i]);
    if (d > worst) worst = d;
  }
  if (max_abs) *max_abs = worst;
  return bad;
}
