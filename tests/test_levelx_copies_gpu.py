"""Omatcopy, Im2col and Col2im on the GPU (through the C ABI) against the CPU oracle, bit for bit where the routine
only moves or scales data.

Grids follow the reference's descriptors (test/routines/levelx/xomatcopy.hpp, xim2col.hpp, xcol2im.hpp)."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("precision", (32, 64, 16, 3232, 6464))
def test_omatcopy(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision)
    trs = (H.NO, H.YES, H.CONJ) if precision > 100 else (H.NO, H.YES)
    for layout, trans, (m, n), off in itertools.product((H.ROW, H.COL), trs, ((7, 64), (64, 7), (100, 33)), (0, 10)):
        a_one, a_two = (n, m) if layout == H.ROW else (m, n)
        b_one, b_two = (a_two, a_one) if trans != H.NO else (a_one, a_two)
        a_ld, b_ld = a_one + 1, b_one + 3
        a = H.rand_buffer(rng, precision, off + a_ld * a_two + H.CANARY)
        b = H.rand_buffer(rng, precision, off + b_ld * b_two + H.CANARY)
        alpha = 3.14 if precision < 100 else 3.14 + 0.5j
        da, db = H.to_device(torch, precision, a), H.to_device(torch, precision, b)
        torch.cuda.synchronize()
        st = cb.Omatcopy(layout, trans, m, n, alpha, da, off, a_ld, db, off, b_ld, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        want = oracle.omatcopy(precision, layout, trans, m, n, alpha, a, off, a_ld, b, off, b_ld)
        got = H.to_host(precision, db)
        if precision < 100:
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (layout, trans, m, n)
        else:  # a complex multiply may be fused differently: rounding level
            eps = 2.0 ** -22 if precision == 3232 else 2.0 ** -51
            assert np.abs(got - want).max() <= eps * 8 * abs(alpha)
            changed = got != b
            rows, cols = (n, m) if trans != H.NO else (m, n)
            assert changed.sum() <= rows * cols


def test_omatcopy_large_runs_near_memory_speed(cuda):
    torch = cuda
    n = 8192
    a = torch.rand(n * n, device="cuda")
    b = torch.empty(n * n, device="cuda")
    torch.cuda.synchronize()
    assert cb.Omatcopy(H.COL, H.YES, n, n, 2.0, a, 0, n, b, 0, n) == 0
    assert torch.equal(b.view(n, n), (a.view(n, n) * 2.0).T.contiguous())


@pytest.mark.parametrize("precision", (32, 64, 16, 3232, 6464))
def test_im2col_and_col2im(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision + 7)
    i = 0
    for mode, pad, dil, ksz, stride, ch in itertools.product((151, 152), (0, 1, 2), (1, 2), (1, 3), (1, 2, 3), (1, 3)):
        h, w = ((7, 8), (8, 5), (13, 9))[i % 3]
        off = (0, 10)[i % 2]
        i += 1
        oh, ow = oracle.conv_output_size(h, w, ksz, ksz + 1, pad, pad, stride, stride, dil, dil)
        im = H.rand_buffer(rng, precision, off + ch * h * w + H.CANARY, -1, 1)
        col = H.rand_buffer(rng, precision, off + ch * ksz * (ksz + 1) * oh * ow + H.CANARY, -1, 1)
        args = (mode, ch, h, w, ksz, ksz + 1, pad, pad, stride, stride, dil, dil)
        dim, dcol = H.to_device(torch, precision, im), H.to_device(torch, precision, col)
        torch.cuda.synchronize()
        assert cb.Im2col(*args, dim, off, dcol, off, precision=precision) == cb.StatusCode.kSuccess
        want = oracle.im2col(*args, im, off, col, off)
        assert np.array_equal(H.to_host(precision, dcol).view(np.uint8), want.view(np.uint8)), ("im2col",) + args
        dim, dcol = H.to_device(torch, precision, im), H.to_device(torch, precision, col)
        torch.cuda.synchronize()
        assert cb.Col2im(*args, dcol, off, dim, off, precision=precision) == cb.StatusCode.kSuccess
        want = oracle.col2im(*args, col, off, im, off)
        got = H.to_host(precision, dim)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), ("col2im",) + args
    assert i == 144


def test_im2col_then_gemm_equals_convgemm(cuda):
    """The two-step method (Im2col, then Gemm with the weights) gives what Convgemm gives in one call."""
    torch = cuda
    rng = np.random.default_rng(3)
    ch, h, w, kh, kw, nk = 16, 20, 24, 3, 3, 32
    oh, ow = oracle.conv_output_size(h, w, kh, kw, 1, 1, 1, 1, 1, 1)
    im = torch.from_numpy(rng.uniform(-1, 1, ch * h * w).astype(np.float32)).cuda()
    ker = torch.from_numpy(rng.uniform(-1, 1, nk * ch * kh * kw).astype(np.float32)).cuda()
    col = torch.zeros(ch * kh * kw * oh * ow, device="cuda")
    two_step = torch.zeros(nk * oh * ow, device="cuda")
    one_step = torch.zeros(nk * oh * ow, device="cuda")
    torch.cuda.synchronize()
    assert cb.Im2col(151, ch, h, w, kh, kw, 1, 1, 1, 1, 1, 1, im, 0, col, 0) == 0
    k = ch * kh * kw
    # result[co][p] = sum_k weights[co][k] * col[k][p]: row-major (nk x k) times (k x oh*ow)
    assert cb.Gemm(H.ROW, H.NO, H.NO, nk, oh * ow, k, 1.0, ker, 0, k, col, 0, oh * ow, 0.0, two_step, 0, oh * ow) == 0
    assert cb.Convgemm(151, ch, h, w, kh, kw, 1, 1, 1, 1, 1, 1, nk, 1, im, 0, ker, 0, one_step, 0) == 0
    assert torch.allclose(two_step, one_step, atol=1e-4, rtol=1e-5)
