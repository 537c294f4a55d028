"""Large complex GEMMs run as a real product of twice the rows and twice the inner dimension on the tensor-core
kernels (csrc/complex_on_real.cpp). Parity against the fp64 oracle on all layouts and transposes (including the
conjugate ones), complex and real scalars, offsets and odd leading dimensions, with the reference's margins
(test/correctness/tester.cpp:29-69) and the tight normalised bounds of the CUDA-core path."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu
TIGHT = {3232: 2.0 ** -19, 6464: 2.0 ** -47}


@pytest.mark.parametrize("precision,shape", ((3232, (512, 512, 512)), (3232, (700, 520, 380)), (6464, (1152, 1152, 128))))
def test_complex_gemm_on_the_real_kernels(cuda, precision, shape):
    torch = cuda
    rng = np.random.default_rng(precision)
    m, n, k = shape
    trs = (H.NO, H.YES, H.CONJ)
    scalars = ((1.5 - 0.5j, 0.5 + 0.25j), (2.0, 0.5), (1.0 + 1.0j, 0.0))
    for i, (layout, ta, tb) in enumerate(itertools.product((H.ROW, H.COL), trs, trs)):
        alpha, beta = scalars[i % 3]
        off = (0, 10, 3)[i % 3]
        pad = (0, 1, 4)[i % 3]
        case = H.gemm_case(rng, precision, layout, ta, tb, m, n, k, off, off, off, (pad, pad, pad), poison_c=(beta == 0.0))
        da, db, dc = (H.to_device(torch, precision, case[x]) for x in "abc")
        torch.cuda.synchronize()
        st = cb.Gemm(layout, ta, tb, m, n, k, alpha, da, off, case["a_ld"], db, off, case["b_ld"], beta, dc, off,
                     case["c_ld"], precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        assert cb.last_kernel().startswith("complex_on_"), cb.last_kernel()
        got = H.to_host(precision, dc)
        c_in = case["c"].copy()
        if beta == 0.0:
            c_in[:] = 0
        want = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alpha, case["a"], off, case["a_ld"], case["b"], off,
                               case["b_ld"], beta, c_in, off, case["c_ld"])
        mask = H.c_mask(layout, m, n, off, case["c_ld"], case["c"].size)
        H.check_against_oracle(precision, got, want, mask, case["c"])
        err = np.abs(oracle.widen(precision, got[mask]) - want[mask]).max() / (8.0 * k * abs(alpha) + 2.0 * abs(beta))
        assert err < TIGHT[precision], (layout, ta, tb, err)


def test_small_complex_gemm_stays_on_the_cuda_cores(cuda):
    torch = cuda
    rng = np.random.default_rng(1)
    case = H.gemm_case(rng, 3232, H.COL, H.NO, H.NO, 64, 64, 64)
    da, db, dc = (H.to_device(torch, 3232, case[x]) for x in "abc")
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, 64, 64, 64, 1.0, da, 0, 64, db, 0, 64, 0.0, dc, 0, 64, precision=3232) == 0
    assert cb.last_kernel().startswith("simt_"), cb.last_kernel()
