"""The level-3 oracle (oracle/level3_oracle.c) against independent numpy evaluations of the BLAS definitions.

The reference's own tests compare Symm ... Trsm with a CBLAS library on seeded data and hold no golden vectors
(test/routines/level3/xsymm.hpp:113-121 and its siblings); numpy's complex128 arithmetic on explicitly built dense
matrices plays that part here, on the reference's size grid {7, 64} with offsets and padded leading dimensions."""
import itertools

import numpy as np
import pytest

from oracle import cpu_oracle as oracle

ROW, COL, NO, YES, CONJ, UPPER, LOWER, NONUNIT, UNIT, LEFT, RIGHT = 101, 102, 111, 112, 113, 121, 122, 131, 132, 141, 142
PRECISIONS = (32, 64, 3232, 6464, 16)


def rand(rng, precision, size):
    x = rng.uniform(-2, 2, size)
    if precision > 100:
        x = x + 1j * rng.uniform(-2, 2, size)
    return x.astype(oracle.NP_OF[precision])


def view(buf, layout, rows, cols, off, ld):
    """(rows x cols matrix stored in buf with the API's addressing, widened; the buffer indices of its elements)."""
    idx = off + (np.arange(rows)[:, None] * ld + np.arange(cols)[None, :] if layout == ROW
                 else np.arange(cols)[None, :] * ld + np.arange(rows)[:, None])
    wide = buf.astype(np.complex128 if np.iscomplexobj(buf) else np.float64)
    return wide[idx], idx


def op(x, trans):
    return x if trans == NO else (x.T if trans == YES else x.conj().T)


def from_triangle(a, triangle, kind, unit=False):
    up = np.triu(a) if triangle == UPPER else np.tril(a)
    if kind == 2:
        if unit:
            np.fill_diagonal(up, 1.0)
        return up
    strict = up - np.diag(np.diag(up))
    d = np.diag(np.diag(up).real) if kind == 1 else np.diag(np.diag(up))
    return strict + d + (strict.conj().T if kind == 1 else strict.T)


def scalars(precision):
    return ((3.14, 0.5), (1.0, 0.0), (0.0, 1.0)) if precision < 100 else ((3.14 + 0.5j, 0.5 - 0.25j), (1.0, 0.0))


@pytest.mark.parametrize("precision", PRECISIONS)
def test_symm_and_hemm(precision):
    rng = np.random.default_rng(precision)
    for herm, layout, side, triangle, (m, n), off in itertools.product(
            (False, True) if precision > 100 else (False,), (ROW, COL), (LEFT, RIGHT), (UPPER, LOWER), ((7, 64), (64, 7), (9, 9)),
            (0, 10)):
        k = m if side == LEFT else n
        a_ld, (b_one, b_two) = k + 3, ((n, m) if layout == ROW else (m, n))
        b_ld, c_ld = b_one + 1, b_one + 2
        a, b, c = rand(rng, precision, off + a_ld * k), rand(rng, precision, off + b_ld * b_two), rand(rng, precision, off + c_ld * b_two)
        for alpha, beta in scalars(precision):
            got = oracle.symm_f64(precision, layout, side, triangle, m, n, alpha, a, off, a_ld, b, off, b_ld, beta, c, off,
                                  c_ld, hermitian=herm)
            A, _ = view(a, layout, k, k, off, a_ld)
            B, _ = view(b, layout, m, n, off, b_ld)
            C, ci = view(c, layout, m, n, off, c_ld)
            S = from_triangle(A, triangle, 1 if herm else 0)
            want = alpha * (S @ B if side == LEFT else B @ S) + beta * C
            assert np.allclose(got[ci], want, rtol=1e-12, atol=1e-12)
            untouched = np.ones(c.size, bool)
            untouched[ci.ravel()] = False
            assert np.array_equal(got[untouched], oracle.widen(precision, c)[untouched])


@pytest.mark.parametrize("precision", PRECISIONS)
def test_rank_k_updates(precision):
    rng = np.random.default_rng(precision + 1)
    for herm, layout, triangle, trans, (n, k), off in itertools.product(
            (False, True) if precision > 100 else (False,), (ROW, COL), (UPPER, LOWER), (NO, YES), ((7, 64), (64, 7)), (0, 10)):
        rows, cols = (n, k) if trans == NO else (k, n)
        one, two = (cols, rows) if layout == ROW else (rows, cols)
        a_ld, b_ld, c_ld = one + 1, one + 2, n + 3
        a, b, c = rand(rng, precision, off + a_ld * two), rand(rng, precision, off + b_ld * two), rand(rng, precision, off + c_ld * n)
        A, _ = view(a, layout, rows, cols, off, a_ld)
        B, _ = view(b, layout, rows, cols, off, b_ld)
        C, ci = view(c, layout, n, n, off, c_ld)
        t = trans if not herm else (NO if trans == NO else CONJ)
        oa, ob = op(A, t), op(B, t)
        tr = (lambda x: x.conj().T) if herm else (lambda x: x.T)
        mask = np.triu(np.ones((n, n), bool)) if triangle == UPPER else np.tril(np.ones((n, n), bool))
        for alpha, beta in scalars(precision):
            if herm:
                beta = float(np.real(beta))
            al1 = float(np.real(alpha)) if herm else alpha
            got = oracle.syrk_f64(precision, layout, triangle, trans, n, k, al1, a, off, a_ld, beta, c, off, c_ld,
                                  hermitian=herm)
            want = al1 * oa @ tr(oa) + beta * C
            if herm:
                want[np.diag_indices(n)] = want[np.diag_indices(n)].real
            assert np.allclose(got[ci][mask], want[mask], rtol=1e-12, atol=1e-12)
            assert np.array_equal(got[ci][~mask], C[~mask])
            got = oracle.syr2k_f64(precision, layout, triangle, trans, n, k, alpha, a, off, a_ld, b, off, b_ld, beta, c,
                                   off, c_ld, hermitian=herm)
            want = alpha * oa @ tr(ob) + (np.conj(alpha) if herm else alpha) * ob @ tr(oa) + beta * C
            if herm:
                want[np.diag_indices(n)] = want[np.diag_indices(n)].real
            assert np.allclose(got[ci][mask], want[mask], rtol=1e-12, atol=1e-12)
            assert np.array_equal(got[ci][~mask], C[~mask])


@pytest.mark.parametrize("precision", (32, 64, 3232, 6464))
def test_trmm_and_trsm(precision):
    rng = np.random.default_rng(precision + 2)
    trs = (NO, YES, CONJ) if precision > 100 else (NO, YES)
    for layout, side, triangle, trans, diag, (m, n) in itertools.product((ROW, COL), (LEFT, RIGHT), (UPPER, LOWER), trs,
                                                                         (NONUNIT, UNIT), ((7, 64), (64, 7))):
        k = m if side == LEFT else n
        off, a_ld = 10, k + 2
        b_one, b_two = (n, m) if layout == ROW else (m, n)
        b_ld = b_one + 1
        # well conditioned also with a unit diagonal: small off-diagonal entries, diagonal away from zero
        a, b = (rand(rng, precision, off + a_ld * k) * 0.05).astype(oracle.NP_OF[precision]), rand(rng, precision, off + b_ld * b_two)
        didx = off + np.arange(k) * (a_ld + 1)
        a[didx] = a[didx] + (2.0 if precision < 100 else 2.0 + 0j)
        A, _ = view(a, layout, k, k, off, a_ld)
        B, bi = view(b, layout, m, n, off, b_ld)
        T = op(from_triangle(A, triangle, 2, diag == UNIT), trans)
        alpha = 1.5 if precision < 100 else 1.5 - 0.5j
        got = oracle.trmm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, off, a_ld, b, off, b_ld)
        want = alpha * (T @ B if side == LEFT else B @ T)
        assert np.allclose(got[bi], want, rtol=1e-12, atol=1e-12)
        got = oracle.trsm_f64(precision, layout, side, triangle, trans, diag, m, n, alpha, a, off, a_ld, b, off, b_ld)
        X = got[bi]
        assert np.allclose(T @ X if side == LEFT else X @ T, alpha * B, rtol=1e-9, atol=1e-9)


def test_data_movement_oracles_on_a_hand_checked_case():
    # 1 channel, 3 x 3 image, 2 x 2 kernel, no padding: four patches
    im = np.arange(9, dtype=np.float32)
    col = oracle.im2col(151, 1, 3, 3, 2, 2, 0, 0, 1, 1, 1, 1, im, 0, np.zeros(16, np.float32), 0)
    assert col.reshape(4, 4).tolist() == [[0, 1, 3, 4], [1, 2, 4, 5], [3, 4, 6, 7], [4, 5, 7, 8]]
    flipped = oracle.im2col(152, 1, 3, 3, 2, 2, 0, 0, 1, 1, 1, 1, im, 0, np.zeros(16, np.float32), 0)
    assert np.array_equal(flipped.reshape(4, 4), col.reshape(4, 4)[::-1])
    back = oracle.col2im(151, 1, 3, 3, 2, 2, 0, 0, 1, 1, 1, 1, np.ones(16, np.float32), 0, np.zeros(9, np.float32), 0)
    assert back.reshape(3, 3).tolist() == [[1, 2, 1], [2, 4, 2], [1, 2, 1]]     # how many patches cover each pixel
    a = np.arange(6, dtype=np.float32)                                             # 2 x 3 row-major
    b = oracle.omatcopy(32, 101, 112, 2, 3, 2.0, a, 0, 3, np.zeros(6, np.float32), 0, 2)
    assert b.reshape(3, 2).tolist() == [[0, 6], [2, 8], [4, 10]]
