"""Status codes that need real device allocations: buffers that are too small, in A, B, C order
(reference: src/utilities/buffer_test.hpp:27-73; TestInvalid in test/correctness/testblas.cpp:280-352)."""
import ctypes

import pytest

import clblast_b200 as cb

pytestmark = pytest.mark.gpu


class RawAlloc:
    """cudaMalloc'ed buffer, so that the allocation's size is exactly what was asked for."""

    def __init__(self, nbytes):
        from cuda.bindings import runtime as rt
        self.rt = rt
        err, self.ptr = rt.cudaMalloc(nbytes)
        assert int(err) == 0

    def free(self):
        self.rt.cudaFree(self.ptr)


def test_insufficient_memory_is_reported_per_matrix(cuda):
    n = 64
    full, short = n * n * 4, (n * n - 1) * 4
    S = cb.StatusCode
    cases = [((short, full, full), S.kInsufficientMemoryA), ((full, short, full), S.kInsufficientMemoryB),
             ((full, full, short), S.kInsufficientMemoryC), ((short, short, short), S.kInsufficientMemoryA),
             ((full, full, full), S.kSuccess)]
    for sizes, expected in cases:
        bufs = [RawAlloc(s) for s in sizes]
        try:
            st = cb.Gemm(102, 111, 111, n, n, n, 1.0, int(bufs[0].ptr), 0, n, int(bufs[1].ptr), 0, n, 0.0,
                         int(bufs[2].ptr), 0, n, precision=32)
            assert st == expected, (sizes, st)
            # an offset pushes an exactly fitting matrix over the end of its buffer
            if expected == S.kSuccess:
                st = cb.Gemm(102, 111, 111, n, n, n, 1.0, int(bufs[0].ptr), 0, n, int(bufs[1].ptr), 1, n, 0.0,
                             int(bufs[2].ptr), 0, n, precision=32)
                assert st == S.kInsufficientMemoryB
        finally:
            for b in bufs:
                b.free()


def test_strided_batched_checks_the_last_batch(cuda):
    n, batch = 16, 3
    per = n * n
    S = cb.StatusCode
    a, b = RawAlloc(per * batch * 4), RawAlloc(per * batch * 4)
    c_ok, c_short = RawAlloc(per * batch * 4), RawAlloc((per * batch - 1) * 4)
    try:
        args = lambda c: (102, 111, 111, n, n, n, 1.0, int(a.ptr), 0, n, per, int(b.ptr), 0, n, per, 0.0, int(c.ptr),
                          0, n, per, batch)
        assert cb.GemmStridedBatched(*args(c_ok), precision=32) == S.kSuccess
        assert cb.GemmStridedBatched(*args(c_short), precision=32) == S.kInsufficientMemoryC
    finally:
        for x in (a, b, c_ok, c_short):
            x.free()


def test_host_pointer_is_an_invalid_matrix(cuda):
    host = (ctypes.c_float * 64)()
    st = cb.Gemm(102, 111, 111, 8, 8, 8, 1.0, ctypes.addressof(host), 0, 8, ctypes.addressof(host), 0, 8, 0.0,
                 ctypes.addressof(host), 0, 8, precision=32)
    assert st == cb.StatusCode.kInvalidMatrixA
