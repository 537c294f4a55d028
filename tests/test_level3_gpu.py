"""Parity of the level-3 routines built on GEMM (Symm, Hemm, Syrk, Herk, Syr2k, Her2k, Trmm, Trsm) on the GPU, through
the C ABI, against the CPU oracle.

Case grids follow the reference's test descriptors (test/routines/level3/xsymm.hpp ... xtrsm.hpp with
test/correctness/testblas.hpp:138-158): sizes {7, 64}, both layouts, sides, triangles, transposes and diagonals,
offsets {0, 10}, padded leading dimensions, canary elements after each buffer; larger shapes are added so that the
inner products reach the tensor-core kernels and Trsm recurses over several diagonal blocks. Tolerances: the
reference's margins (test/correctness/tester.cpp:29-69) against the fp64 oracle, plus a normalised bound."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu

UPPER, LOWER, NONUNIT, UNIT, LEFT, RIGHT = 121, 122, 131, 132, 141, 142
TIGHT = {32: 2.0 ** -19, 64: 2.0 ** -47, 16: 4e-3, 3232: 2.0 ** -18, 6464: 2.0 ** -46}


def scalars(precision):
    return ((3.14, 0.5), (1.0, 0.0)) if precision < 100 else ((3.14 + 0.5j, 0.5 - 0.25j), (1.0, 0.0))


def footprint(layout, rows, cols, off, ld, size):
    return H.c_mask(layout, rows, cols, off, ld, size)


def check(precision, got, want, mask, before, scale):
    H.check_against_oracle(precision, got, want, mask, before)
    err = np.abs(oracle.widen(precision, got[mask]) - want[mask]).max() / scale
    assert err < TIGHT[precision], f"normalised error {err:.3e}"


@pytest.mark.parametrize("precision", (32, 64, 16, 3232, 6464))
def test_symm_and_hemm(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision)
    variants = (False, True) if precision > 100 else (False,)
    shapes = ((7, 64), (64, 7), (64, 64), (300, 520))
    for herm, layout, side, triangle, (m, n) in itertools.product(variants, (H.ROW, H.COL), (LEFT, RIGHT), (UPPER, LOWER),
                                                                 shapes):
        off = 10 if m == 7 else 0
        k = m if side == LEFT else n
        b_one, b_two = (n, m) if layout == H.ROW else (m, n)
        a_ld, b_ld, c_ld = k + 1, b_one + 2, b_one + 3
        a = H.rand_buffer(rng, precision, off + a_ld * k + H.CANARY)
        b = H.rand_buffer(rng, precision, off + b_ld * b_two + H.CANARY)
        c = H.rand_buffer(rng, precision, off + c_ld * b_two + H.CANARY)
        alpha, beta = scalars(precision)[(m + n) % 2]
        da, db, dc = (H.to_device(torch, precision, x) for x in (a, b, c))
        torch.cuda.synchronize()
        fn = cb.Hemm if herm else cb.Symm
        st = fn(layout, side, triangle, m, n, alpha, da, off, a_ld, db, off, b_ld, beta, dc, off, c_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.symm_f64(precision, layout, side, triangle, m, n, alpha, a, off, a_ld, b, off, b_ld, beta, c, off,
                               c_ld, hermitian=herm)
        mask = footprint(layout, m, n, off, c_ld, c.size)
        check(precision, H.to_host(precision, dc), want, mask, c, (8.0 if precision > 100 else 4.0) * k * abs(alpha) + 2 * abs(beta) + 1e-30)


@pytest.mark.parametrize("precision", (32, 64, 16, 3232, 6464))
def test_syrk_herk_syr2k_her2k(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision + 1)
    variants = (False, True) if precision > 100 else (False,)
    shapes = ((7, 64), (64, 7), (64, 64), (300, 200), (129, 257))
    for herm, layout, triangle, trans, (n, k) in itertools.product(variants, (H.ROW, H.COL), (UPPER, LOWER), (H.NO, H.YES),
                                                                  shapes):
        off = 10 if n == 7 else 0
        rows, cols = (n, k) if trans == H.NO else (k, n)
        one, two = (cols, rows) if layout == H.ROW else (rows, cols)
        a_ld, b_ld, c_ld = one + 1, one + 2, n + 3
        a = H.rand_buffer(rng, precision, off + a_ld * two + H.CANARY)
        b = H.rand_buffer(rng, precision, off + b_ld * two + H.CANARY)
        c = H.rand_buffer(rng, precision, off + c_ld * n + H.CANARY)
        alpha, beta = scalars(precision)[(n + k) % 2]
        if herm:
            beta = float(np.real(beta))
        da, db = H.to_device(torch, precision, a), H.to_device(torch, precision, b)
        scale = (8.0 if precision > 100 else 4.0) * k * abs(alpha) * 2 + 2 * abs(beta) + 1e-30
        # the update touches one triangle of the n x n footprint only
        tri = np.triu(np.ones((n, n), bool)) if triangle == UPPER else np.tril(np.ones((n, n), bool))
        idx = off + (np.arange(n)[:, None] * c_ld + np.arange(n)[None, :] if layout == H.ROW
                     else np.arange(n)[None, :] * c_ld + np.arange(n)[:, None])
        mask = np.zeros(c.size, bool)
        mask[idx[tri]] = True

        dc = H.to_device(torch, precision, c)
        torch.cuda.synchronize()
        al1 = float(np.real(alpha)) if herm else alpha
        fn = cb.Herk if herm else cb.Syrk
        st = fn(layout, triangle, trans, n, k, al1, da, off, a_ld, beta, dc, off, c_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.syrk_f64(precision, layout, triangle, trans, n, k, al1, a, off, a_ld, beta, c, off, c_ld, hermitian=herm)
        check(precision, H.to_host(precision, dc), want, mask, c, scale)

        dc = H.to_device(torch, precision, c)
        torch.cuda.synchronize()
        fn = cb.Her2k if herm else cb.Syr2k
        st = fn(layout, triangle, trans, n, k, alpha, da, off, a_ld, db, off, b_ld, beta, dc, off, c_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.syr2k_f64(precision, layout, triangle, trans, n, k, alpha, a, off, a_ld, b, off, b_ld, beta, c, off,
                                c_ld, hermitian=herm)
        check(precision, H.to_host(precision, dc), want, mask, c, scale)


def triangular_case(rng, precision, k, off, a_ld):
    """A triangular operand whose solves are well conditioned with and without a unit diagonal."""
    a = (H.rand_buffer(rng, precision, off + a_ld * k + H.CANARY) * 0.05).astype(H.NP_OF[precision])
    d = off + np.arange(k) * (a_ld + 1)
    a[d] = a[d] + H.NP_OF[precision](2.0)
    return a


@pytest.mark.parametrize("precision", (32, 64, 16, 3232, 6464))
def test_trmm(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision + 2)
    trs = (H.NO, H.YES, H.CONJ) if precision > 100 else (H.NO, H.YES)
    for layout, side, triangle, trans, diag, (m, n) in itertools.product((H.ROW, H.COL), (LEFT, RIGHT), (UPPER, LOWER), trs,
                                                                         (NONUNIT, UNIT), ((7, 64), (64, 7), (260, 300))):
        off = 10 if m == 7 else 0
        k = m if side == LEFT else n
        b_one, b_two = (n, m) if layout == H.ROW else (m, n)
        a_ld, b_ld = k + 1, b_one + 2
        a = triangular_case(rng, precision, k, off, a_ld)
        b = H.rand_buffer(rng, precision, off + b_ld * b_two + H.CANARY)
        alpha = 1.5 if precision < 100 else 1.5 - 0.5j
        da, db = H.to_device(torch, precision, a), H.to_device(torch, precision, b)
        torch.cuda.synchronize()
        st = cb.Trmm(layout, side, triangle, trans, diag, m, n, alpha, da, off, a_ld, db, off, b_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.trmm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, off, a_ld, b, off, b_ld)
        mask = footprint(layout, m, n, off, b_ld, b.size)
        check(precision, H.to_host(precision, db), want, mask, b, 8.0 * abs(alpha) * (2.0 + 0.1 * k) + 1e-30)


@pytest.mark.parametrize("precision", (32, 64, 3232, 6464))
def test_trsm(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision + 3)
    trs = (H.NO, H.YES, H.CONJ) if precision > 100 else (H.NO, H.YES)
    # 7 and 64: the reference's grid; 130 and 200: three and four diagonal blocks with a ragged last one
    for layout, side, triangle, trans, diag, (m, n) in itertools.product((H.ROW, H.COL), (LEFT, RIGHT), (UPPER, LOWER), trs,
                                                                         (NONUNIT, UNIT), ((7, 64), (64, 7), (130, 200))):
        off = 10 if m == 7 else 0
        k = m if side == LEFT else n
        b_one, b_two = (n, m) if layout == H.ROW else (m, n)
        a_ld, b_ld = k + 1, b_one + 2
        a = triangular_case(rng, precision, k, off, a_ld)
        b = H.rand_buffer(rng, precision, off + b_ld * b_two + H.CANARY)
        alpha = 1.5 if precision < 100 else 1.5 - 0.5j
        da, db = H.to_device(torch, precision, a), H.to_device(torch, precision, b)
        torch.cuda.synchronize()
        st = cb.Trsm(layout, side, triangle, trans, diag, m, n, alpha, da, off, a_ld, db, off, b_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.trsm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, off, a_ld, b, off, b_ld)
        mask = footprint(layout, m, n, off, b_ld, b.size)
        got = H.to_host(precision, db)
        H.check_against_oracle(precision, got, want, mask, b)
        err = np.abs(oracle.widen(precision, got[mask]) - want[mask]).max() / np.abs(want[mask]).max()
        assert err < (1e-4 if precision in (32, 3232) else 1e-12), err


def test_large_trsm_and_syrk_reach_the_tensor_cores(cuda):
    """A 2048-wide solve: the updates between diagonal blocks are large GEMMs on the tensor-core kernels; the result is
    checked through the residual op(A) X - alpha B, which needs no host solve."""
    torch = cuda
    n = 2048
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.rand(n * n, generator=g, device="cuda") * 0.02 - 0.01
    a.view(n, n).diagonal().add_(1.0)
    b = torch.rand(n * n, generator=g, device="cuda") * 2 - 1
    x = b.clone()
    torch.cuda.synchronize()
    assert cb.Trsm(H.COL, LEFT, LOWER, H.NO, NONUNIT, n, n, 1.0, a, 0, n, x, 0, n) == 0
    L = torch.tril(a.view(n, n).T.double())          # column-major storage seen as a row-major transpose
    resid = (L @ x.view(n, n).T.double() - b.view(n, n).T.double()).abs().max().item()
    assert resid < 1e-3, resid
    c = torch.zeros(n * n, device="cuda")
    torch.cuda.synchronize()
    assert cb.Syrk(H.COL, LOWER, H.NO, n, n, 1.0, b, 0, n, 0.0, c, 0, n) == 0
    B = b.view(n, n).T.double()
    want = torch.tril(B @ B.T)
    # k-ascending fp32 accumulation of 2048 terms (the diagonal sums squares, all of one sign): 2^-18 of sum |a||b|
    assert ((torch.tril(c.view(n, n).T.double()) - want).abs().max() / n).item() < 2.0 ** -18
    assert float(torch.triu(c.view(n, n).T, 1).abs().max()) == 0.0   # the other triangle is untouched


def test_argument_checks_follow_the_reference_order(cuda):
    from tests.test_errors_gpu import RawAlloc
    torch = cuda
    buf = torch.zeros(64 * 64, device="cuda")
    raw = RawAlloc(8 * 4)      # cudaMalloc'ed, so the allocation really ends after 8 floats
    small = int(raw.ptr)
    S = cb.StatusCode
    kw = dict(precision=32)
    assert cb.Symm(H.COL, LEFT, UPPER, 0, 4, 1.0, buf, 0, 4, buf, 0, 4, 0.0, buf, 0, 4) == S.kInvalidDimension
    assert cb.Symm(H.COL, LEFT, UPPER, 8, 8, 1.0, buf, 0, 7, buf, 0, 8, 0.0, buf, 0, 8) == S.kInvalidLeadDimA
    assert cb.Symm(H.COL, LEFT, UPPER, 8, 8, 1.0, buf, 0, 8, buf, 0, 7, 0.0, buf, 0, 8) == S.kInvalidLeadDimB
    assert cb.Symm(H.COL, LEFT, UPPER, 8, 8, 1.0, buf, 0, 8, buf, 0, 8, 0.0, small, 0, 8, **kw) == S.kInsufficientMemoryC
    assert cb.Syrk(H.COL, UPPER, H.NO, 8, 0, 1.0, buf, 0, 8, 0.0, buf, 0, 8) == S.kInvalidDimension
    assert cb.Syrk(H.COL, UPPER, H.NO, 8, 8, 1.0, small, 0, 8, 0.0, buf, 0, 8, **kw) == S.kInsufficientMemoryA
    assert cb.Syrk(H.COL, UPPER, H.NO, 8, 8, 1.0, buf, 0, 8, 0.0, buf, 0, 7) == S.kInvalidLeadDimC
    assert cb.Trmm(H.COL, LEFT, UPPER, H.NO, NONUNIT, 8, 0, 1.0, buf, 0, 8, buf, 0, 8) == S.kInvalidDimension
    assert cb.Trsm(H.COL, LEFT, UPPER, H.NO, NONUNIT, 8, 8, 1.0, buf, 0, 8, small, 0, 8, **kw) == S.kInsufficientMemoryB
    assert cb.Trsm(H.ROW, LEFT, UPPER, H.NO, NONUNIT, 8, 8, 1.0, buf, 0, 7, buf, 0, 8) == S.kInvalidLeadDimA
    raw.free()


@pytest.mark.parametrize("precision,n,k,kernel", ((32, 3072, 384, "tc_f32_3xtf32_pair"), (64, 1536, 200, "dmma_f64")))
def test_rank_k_updates_on_the_tensor_core_kernels(cuda, precision, n, k, kernel):
    """Large Syrk / Syr2k run on the tensor-core GEMM kernels, which number only the tiles that touch the triangle and
    mask the diagonal tiles; checked against fp64 products on the device, including that the other triangle and the
    padding between columns keep their old contents."""
    torch = cuda
    dt = torch.float32 if precision == 32 else torch.float64
    g = torch.Generator(device="cuda").manual_seed(n)
    ldc = n + 4
    for layout, triangle, trans in itertools.product((H.ROW, H.COL), (UPPER, LOWER), (H.NO, H.YES)):
        a = (torch.rand(n * k, generator=g, device="cuda", dtype=dt) * 2 - 1)
        b = (torch.rand(n * k, generator=g, device="cuda", dtype=dt) * 2 - 1)
        c0 = (torch.rand(ldc * n, generator=g, device="cuda", dtype=dt) * 2 - 1)
        c = c0.clone()
        # the stored matrix is n x k when (row-major, not transposed) or (column-major, transposed) is read row by row
        rows_first = (layout == H.ROW) == (trans == H.NO)
        a_ld = k if rows_first else n
        A = a.view(n, k).double() if rows_first else a.view(k, n).double().T       # op(A): n x k
        B = b.view(n, k).double() if rows_first else b.view(k, n).double().T
        torch.cuda.synchronize()
        assert cb.Syr2k(layout, triangle, trans, n, k, 1.5, a, 0, a_ld, b, 0, a_ld, 0.5, c, 0, ldc) == 0
        assert kernel in cb.last_kernel(), cb.last_kernel()
        want = 1.5 * (A @ B.T + B @ A.T)
        C0 = c0.view(n, ldc)[:, :n].double()
        C = c.view(n, ldc)[:, :n].double()
        if layout == H.COL:                      # memory rows are columns of C
            C0, C = C0.T, C.T
        keep = torch.triu(torch.ones(n, n, dtype=torch.bool, device="cuda")) if triangle == UPPER else \
            torch.tril(torch.ones(n, n, dtype=torch.bool, device="cuda"))
        err = ((C - (want + 0.5 * C0)).abs()[keep].max() / (3.0 * k + 0.5)).item()
        assert err < (2.0 ** -20 if precision == 32 else 2.0 ** -48), err
        assert torch.equal(C[~keep], C0[~keep])
        assert torch.equal(c.view(n, ldc)[:, n:], c0.view(n, ldc)[:, n:])
