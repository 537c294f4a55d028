// Host-pointer layer (include/b200blas_netlib.h): device buffers sized as the reference sizes them
// (src/clblast_netlib_c.cpp:2718-2749), host to device copies, the device routine through the flat C ABI, and the
// copy of the result back. Everything runs on the library's synchronous path of the current device.
#include "b200blas_netlib.h"

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#include "b200blas.h"

namespace {

void check(int status) {
  if (status != 0) throw std::runtime_error("CLBlast returned with error code " + std::to_string(status));
}
void check(cudaError_t e) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA error: ") + cudaGetErrorString(e));
}

// Device copy of a host matrix; written back on request, released at scope end.
class DeviceCopy {
 public:
  DeviceCopy(const void* host, size_t bytes) : bytes_(bytes) {
    check(cudaMalloc(&ptr_, bytes ? bytes : 1));
    if (bytes) check(cudaMemcpy(ptr_, host, bytes, cudaMemcpyHostToDevice));
  }
  ~DeviceCopy() { cudaFree(ptr_); }
  void read_back(void* host) const { check(cudaMemcpy(host, ptr_, bytes_, cudaMemcpyDeviceToHost)); }
  void* get() const { return ptr_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_;
};

}  // namespace

extern "C" void cblas_sgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const int m, const int n, const int k, const float alpha, const float* a, const int a_ld, const
    float* b, const int b_ld, const float beta, float* c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo), b_rot = (layout == CLBlastLayoutRowMajor) == (b_transpose == CLBlastTransposeNo);
  const size_t a_size = (a_rot ? m : k) * static_cast<size_t>(a_ld), b_size = (b_rot ? k : n) * static_cast<size_t>(b_ld);
  const size_t c_size = ((layout == CLBlastLayoutRowMajor) ? m : n) * static_cast<size_t>(c_ld);
  DeviceCopy da(a, a_size * 4), db(b, b_size * 4), dc(c, c_size * 4);
  check(b200blas_gemm(32, layout, a_transpose, b_transpose, m, n, k, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_dgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const int m, const int n, const int k, const double alpha, const double* a, const int a_ld, const
    double* b, const int b_ld, const double beta, double* c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo), b_rot = (layout == CLBlastLayoutRowMajor) == (b_transpose == CLBlastTransposeNo);
  const size_t a_size = (a_rot ? m : k) * static_cast<size_t>(a_ld), b_size = (b_rot ? k : n) * static_cast<size_t>(b_ld);
  const size_t c_size = ((layout == CLBlastLayoutRowMajor) ? m : n) * static_cast<size_t>(c_ld);
  DeviceCopy da(a, a_size * 8), db(b, b_size * 8), dc(c, c_size * 8);
  check(b200blas_gemm(64, layout, a_transpose, b_transpose, m, n, k, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_cgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const int m, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void*
    b, const int b_ld, const void* beta, void* c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo), b_rot = (layout == CLBlastLayoutRowMajor) == (b_transpose == CLBlastTransposeNo);
  const size_t a_size = (a_rot ? m : k) * static_cast<size_t>(a_ld), b_size = (b_rot ? k : n) * static_cast<size_t>(b_ld);
  const size_t c_size = ((layout == CLBlastLayoutRowMajor) ? m : n) * static_cast<size_t>(c_ld);
  DeviceCopy da(a, a_size * 8), db(b, b_size * 8), dc(c, c_size * 8);
  check(b200blas_gemm(3232, layout, a_transpose, b_transpose, m, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zgemm(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const CLBlastTranspose
    b_transpose, const int m, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void*
    b, const int b_ld, const void* beta, void* c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo), b_rot = (layout == CLBlastLayoutRowMajor) == (b_transpose == CLBlastTransposeNo);
  const size_t a_size = (a_rot ? m : k) * static_cast<size_t>(a_ld), b_size = (b_rot ? k : n) * static_cast<size_t>(b_ld);
  const size_t c_size = ((layout == CLBlastLayoutRowMajor) ? m : n) * static_cast<size_t>(c_ld);
  DeviceCopy da(a, a_size * 16), db(b, b_size * 16), dc(c, c_size * 16);
  check(b200blas_gemm(6464, layout, a_transpose, b_transpose, m, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_ssymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const float alpha, const float* a, const int a_ld, const float* b, const int b_ld, const float
    beta, float* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 4), db(b, lines_bc * b_ld * 4), dc(c, lines_bc * c_ld * 4);
  check(b200blas_symm(32, layout, side, triangle, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_dsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const double alpha, const double* a, const int a_ld, const double* b, const int b_ld, const
    double beta, double* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, lines_bc * b_ld * 8), dc(c, lines_bc * c_ld * 8);
  check(b200blas_symm(64, layout, side, triangle, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_csymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void*
    beta, void* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, lines_bc * b_ld * 8), dc(c, lines_bc * c_ld * 8);
  check(b200blas_symm(3232, layout, side, triangle, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zsymm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void*
    beta, void* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 16), db(b, lines_bc * b_ld * 16), dc(c, lines_bc * c_ld * 16);
  check(b200blas_symm(6464, layout, side, triangle, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_chemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void*
    beta, void* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, lines_bc * b_ld * 8), dc(c, lines_bc * c_ld * 8);
  check(b200blas_hemm(3232, layout, side, triangle, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zhemm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    int m, const int n, const void* alpha, const void* a, const int a_ld, const void* b, const int b_ld, const void*
    beta, void* c, const int c_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, lines_bc = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 16), db(b, lines_bc * b_ld * 16), dc(c, lines_bc * c_ld * 16);
  check(b200blas_hemm(6464, layout, side, triangle, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_ssyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const float alpha, const float* a, const int a_ld, const float beta, float*
    c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 4), dc(c, static_cast<size_t>(n) * c_ld * 4);
  check(b200blas_syrk(32, layout, triangle, a_transpose, n, k, &alpha, da.get(), 0, a_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_dsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const double alpha, const double* a, const int a_ld, const double beta,
    double* c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_syrk(64, layout, triangle, a_transpose, n, k, &alpha, da.get(), 0, a_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_csyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* beta, void*
    c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_syrk(3232, layout, triangle, a_transpose, n, k, alpha, da.get(), 0, a_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zsyrk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* beta, void*
    c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 16), dc(c, static_cast<size_t>(n) * c_ld * 16);
  check(b200blas_syrk(6464, layout, triangle, a_transpose, n, k, alpha, da.get(), 0, a_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_cherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const float alpha, const void* a, const int a_ld, const float beta, void*
    c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_herk(3232, layout, triangle, a_transpose, n, k, &alpha, da.get(), 0, a_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zherk(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    a_transpose, const int n, const int k, const double alpha, const void* a, const int a_ld, const double beta, void*
    c, const int c_ld) {
  const bool a_rot = (layout == CLBlastLayoutRowMajor) == (a_transpose == CLBlastTransposeNo);
  DeviceCopy da(a, (a_rot ? n : k) * static_cast<size_t>(a_ld) * 16), dc(c, static_cast<size_t>(n) * c_ld * 16);
  check(b200blas_herk(6464, layout, triangle, a_transpose, n, k, &alpha, da.get(), 0, a_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_ssyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const float alpha, const float* a, const int a_ld, const float* b, const
    int b_ld, const float beta, float* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 4), db(b, ab_lines * b_ld * 4), dc(c, static_cast<size_t>(n) * c_ld * 4);
  check(b200blas_syr2k(32, layout, triangle, ab_transpose, n, k, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_dsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const double alpha, const double* a, const int a_ld, const double* b,
    const int b_ld, const double beta, double* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 8), db(b, ab_lines * b_ld * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_syr2k(64, layout, triangle, ab_transpose, n, k, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_csyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const void* beta, void* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 8), db(b, ab_lines * b_ld * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_syr2k(3232, layout, triangle, ab_transpose, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zsyr2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const void* beta, void* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 16), db(b, ab_lines * b_ld * 16), dc(c, static_cast<size_t>(n) * c_ld * 16);
  check(b200blas_syr2k(6464, layout, triangle, ab_transpose, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_cher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const float beta, void* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 8), db(b, ab_lines * b_ld * 8), dc(c, static_cast<size_t>(n) * c_ld * 8);
  check(b200blas_her2k(3232, layout, triangle, ab_transpose, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_zher2k(const CLBlastLayout layout, const CLBlastTriangle triangle, const CLBlastTranspose
    ab_transpose, const int n, const int k, const void* alpha, const void* a, const int a_ld, const void* b, const int
    b_ld, const double beta, void* c, const int c_ld) {
  const bool rot = (layout == CLBlastLayoutRowMajor) == (ab_transpose == CLBlastTransposeNo);
  const size_t ab_lines = rot ? n : k;
  DeviceCopy da(a, ab_lines * a_ld * 16), db(b, ab_lines * b_ld * 16), dc(c, static_cast<size_t>(n) * c_ld * 16);
  check(b200blas_her2k(6464, layout, triangle, ab_transpose, n, k, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, &beta, dc.get(), 0, c_ld, 0, 0));
  dc.read_back(c);
}

extern "C" void cblas_strmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const float alpha, const
    float* a, const int a_ld, float* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 4), db(b, b_lines * b_ld * 4);
  check(b200blas_trmm(32, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_dtrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const double alpha, const
    double* a, const int a_ld, double* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_trmm(64, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_ctrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_trmm(3232, layout, side, triangle, a_transpose, diagonal, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_ztrmm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 16), db(b, b_lines * b_ld * 16);
  check(b200blas_trmm(6464, layout, side, triangle, a_transpose, diagonal, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_strsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const float alpha, const
    float* a, const int a_ld, float* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 4), db(b, b_lines * b_ld * 4);
  check(b200blas_trsm(32, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_dtrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const double alpha, const
    double* a, const int a_ld, double* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_trsm(64, layout, side, triangle, a_transpose, diagonal, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_ctrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_trsm(3232, layout, side, triangle, a_transpose, diagonal, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_ztrsm(const CLBlastLayout layout, const CLBlastSide side, const CLBlastTriangle triangle, const
    CLBlastTranspose a_transpose, const CLBlastDiagonal diagonal, const int m, const int n, const void* alpha, const
    void* a, const int a_ld, void* b, const int b_ld) {
  const size_t k = side == CLBlastSideLeft ? m : n, b_lines = (layout == CLBlastLayoutRowMajor) ? m : n;
  DeviceCopy da(a, k * a_ld * 16), db(b, b_lines * b_ld * 16);
  check(b200blas_trsm(6464, layout, side, triangle, a_transpose, diagonal, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_somatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int
    n, const float alpha, const float* a, const int a_ld, float* b, const int b_ld) {
  const size_t a_lines = (layout == CLBlastLayoutRowMajor) ? m : n, a_one = (layout == CLBlastLayoutRowMajor) ? n : m;
  const size_t b_lines = a_transpose != CLBlastTransposeNo ? a_one : a_lines;
  DeviceCopy da(a, a_lines * a_ld * 4), db(b, b_lines * b_ld * 4);
  check(b200blas_omatcopy(32, layout, a_transpose, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_domatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int
    n, const double alpha, const double* a, const int a_ld, double* b, const int b_ld) {
  const size_t a_lines = (layout == CLBlastLayoutRowMajor) ? m : n, a_one = (layout == CLBlastLayoutRowMajor) ? n : m;
  const size_t b_lines = a_transpose != CLBlastTransposeNo ? a_one : a_lines;
  DeviceCopy da(a, a_lines * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_omatcopy(64, layout, a_transpose, m, n, &alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_comatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int
    n, const void* alpha, const void* a, const int a_ld, void* b, const int b_ld) {
  const size_t a_lines = (layout == CLBlastLayoutRowMajor) ? m : n, a_one = (layout == CLBlastLayoutRowMajor) ? n : m;
  const size_t b_lines = a_transpose != CLBlastTransposeNo ? a_one : a_lines;
  DeviceCopy da(a, a_lines * a_ld * 8), db(b, b_lines * b_ld * 8);
  check(b200blas_omatcopy(3232, layout, a_transpose, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}

extern "C" void cblas_zomatcopy(const CLBlastLayout layout, const CLBlastTranspose a_transpose, const int m, const int
    n, const void* alpha, const void* a, const int a_ld, void* b, const int b_ld) {
  const size_t a_lines = (layout == CLBlastLayoutRowMajor) ? m : n, a_one = (layout == CLBlastLayoutRowMajor) ? n : m;
  const size_t b_lines = a_transpose != CLBlastTransposeNo ? a_one : a_lines;
  DeviceCopy da(a, a_lines * a_ld * 16), db(b, b_lines * b_ld * 16);
  check(b200blas_omatcopy(6464, layout, a_transpose, m, n, alpha, da.get(), 0, a_ld, db.get(), 0, b_ld, 0, 0));
  db.read_back(b);
}
