"""The C interface (include/b200blas_c.h, named as the reference's C API names its routines) and the host-pointer layer
(include/b200blas_netlib.h, named as the reference's Netlib layer) on the GPU, called through ctypes like a C program
would, against numpy."""
import ctypes

import numpy as np
import pytest

import clblast_b200 as cb
from tests import harness as H

pytestmark = pytest.mark.gpu


class ComplexFloat(ctypes.Structure):
    _fields_ = [("re", ctypes.c_float), ("im", ctypes.c_float)]


def test_c_api_sgemm_and_cgemm(cuda):
    torch = cuda
    L = cb.lib()
    rng = np.random.default_rng(0)
    m, n, k = 48, 40, 56
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    b = rng.uniform(-1, 1, (k, n)).astype(np.float32)
    c = rng.uniform(-1, 1, (m, n)).astype(np.float32)
    da, db, dc = (torch.from_numpy(x).cuda() for x in (a, b, c))
    torch.cuda.synchronize()
    sz, f = ctypes.c_size_t, ctypes.c_float
    L.CLBlastSgemm.restype = ctypes.c_int
    L.CLBlastSgemm.argtypes = [ctypes.c_int] * 3 + [sz] * 3 + [f, ctypes.c_uint64, sz, sz, ctypes.c_uint64, sz, sz, f,
                                                                  ctypes.c_uint64, sz, sz, ctypes.c_void_p, ctypes.c_int]
    st = L.CLBlastSgemm(101, 111, 111, m, n, k, 1.5, da.data_ptr(), 0, k, db.data_ptr(), 0, n, 0.5, dc.data_ptr(), 0, n,
                        None, 0)
    assert st == 0
    assert np.allclose(dc.cpu().numpy(), 1.5 * a @ b + 0.5 * c, atol=1e-4)

    az = (a[:, :n] + 1j * a[:, :n][::-1]).astype(np.complex64)[:n]          # n x n complex
    bz = (b[:n, :n] - 1j * b[:n, :n].T).astype(np.complex64)
    cz = np.zeros((n, n), np.complex64)
    dz = [torch.from_numpy(x).cuda() for x in (az, bz, cz)]
    torch.cuda.synchronize()
    L.CLBlastCgemm.restype = ctypes.c_int
    L.CLBlastCgemm.argtypes = [ctypes.c_int] * 3 + [sz] * 3 + [ComplexFloat, ctypes.c_uint64, sz, sz, ctypes.c_uint64, sz,
                                                                  sz, ComplexFloat, ctypes.c_uint64, sz, sz,
                                                                  ctypes.c_void_p, ctypes.c_int]
    st = L.CLBlastCgemm(101, 111, 113, n, n, n, ComplexFloat(1.0, -2.0), dz[0].data_ptr(), 0, n, dz[1].data_ptr(), 0, n,
                        ComplexFloat(0.0, 0.0), dz[2].data_ptr(), 0, n, None, 0)
    assert st == 0
    assert np.allclose(dz[2].cpu().numpy(), (1 - 2j) * az @ bz.conj().T, atol=1e-3)
    # a zero dimension comes back as the reference's status code
    assert L.CLBlastSgemm(101, 111, 111, 0, n, k, 1.0, da.data_ptr(), 0, k, db.data_ptr(), 0, n, 0.0, dc.data_ptr(), 0, n,
                          None, 0) == cb.StatusCode.kInvalidDimension


def test_host_pointer_layer(cuda):
    L = cb.lib()
    rng = np.random.default_rng(1)
    m, n, k = 33, 20, 47
    a = rng.uniform(-1, 1, (m, k))
    b = rng.uniform(-1, 1, (k, n))
    c = rng.uniform(-1, 1, (m, n))
    want = 0.7 * a @ b + 0.3 * c
    i, d, vp = ctypes.c_int, ctypes.c_double, ctypes.c_void_p
    L.cblas_dgemm.restype = None
    L.cblas_dgemm.argtypes = [i] * 6 + [d, vp, i, vp, i, d, vp, i]
    L.cblas_dgemm(101, 111, 111, m, n, k, 0.7, a.ctypes.data, k, b.ctypes.data, n, 0.3, c.ctypes.data, n)
    assert np.allclose(c, want, atol=1e-12)

    # triangular solve, column-major (numpy arrays transposed in memory), then multiply back
    t = np.tril(rng.uniform(-0.1, 0.1, (m, m))) + 2 * np.eye(m)
    rhs = rng.uniform(-1, 1, (m, n))
    t_cm, x_cm = np.asfortranarray(t), np.asfortranarray(rhs.copy())
    L.cblas_dtrsm.restype = None
    L.cblas_dtrsm.argtypes = [i] * 7 + [d, vp, i, vp, i]
    L.cblas_dtrsm(102, 141, 122, 111, 131, m, n, 1.0, t_cm.ctypes.data, m, x_cm.ctypes.data, m)
    assert np.allclose(t @ x_cm, rhs, atol=1e-10)
    L.cblas_dtrmm.restype = None
    L.cblas_dtrmm.argtypes = L.cblas_dtrsm.argtypes
    L.cblas_dtrmm(102, 141, 122, 111, 131, m, n, 1.0, t_cm.ctypes.data, m, x_cm.ctypes.data, m)
    assert np.allclose(x_cm, rhs, atol=1e-10)

    # complex rank-k update with real scalars
    az = (rng.uniform(-1, 1, (n, k)) + 1j * rng.uniform(-1, 1, (n, k))).astype(np.complex64)
    cz = np.zeros((n, n), np.complex64)
    f = ctypes.c_float
    L.cblas_cherk.restype = None
    L.cblas_cherk.argtypes = [i] * 5 + [f, vp, i, f, vp, i]
    L.cblas_cherk(101, 121, 111, n, k, 2.0, az.ctypes.data, k, 0.0, cz.ctypes.data, n)
    want = 2.0 * az @ az.conj().T
    assert np.allclose(np.triu(cz), np.triu(want), atol=1e-3) and np.all(np.tril(cz, -1) == 0)
