"""The tensor-core HGEMM kernel (TMA + tcgen05 + TMEM) against the fp64 oracle.

Tolerance: the reference's half margins (relative 8e-2 or absolute 0.15, test/correctness/tester.cpp:38-55) against
the fp64 product, and the tight bound |x - r| <= 1e-3 * sum_k|a||b| that fp32 accumulation with one final rounding
to half satisfies (the reference itself accumulates in half and is about 70x less accurate at K = 8192)."""
import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu


def run_tc(torch, rng, layout, ta, tb, m, n, k, alpha, beta, offs=(0, 0, 0), pad=(0, 0, 0), expect_tc=True):
    case = H.gemm_case(rng, 16, layout, ta, tb, m, n, k, offs[0], offs[1], offs[2], pad, lo=-1, hi=1,
                       poison_c=(beta == 0))
    da, db, dc = (H.to_device(torch, 16, case[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.Gemm(layout, ta, tb, m, n, k, alpha, da, offs[0], case["a_ld"], db, offs[1], case["b_ld"], beta, dc, offs[2],
                 case["c_ld"], precision=16)
    assert st == cb.StatusCode.kSuccess, st
    assert cb.last_kernel().startswith("tc_") == expect_tc, cb.last_kernel()
    got = H.to_host(16, dc)
    c_in = case["c"].copy()
    if beta == 0:
        c_in[:] = 0
    want = oracle.gemm_f64(16, layout, ta, tb, m, n, k, alpha, case["a"], offs[0], case["a_ld"], case["b"], offs[1],
                           case["b_ld"], beta, c_in, offs[2], case["c_ld"])
    mask = H.c_mask(layout, m, n, offs[2], case["c_ld"], case["c"].size)
    worst = H.check_against_oracle(16, got, want, mask, case["c"])
    assert worst <= 1e-3 * (abs(alpha) * k + abs(beta)) + 1e-6
    return worst


# every layout / transpose combination: K-contiguous operands are loaded as K-major tiles, the others as MN-major
# column blocks
TC_LAYOUTS = tuple((layout, ta, tb) for layout in (H.ROW, H.COL) for ta in (H.NO, H.YES) for tb in (H.NO, H.YES))


@pytest.mark.parametrize("layout,ta,tb", TC_LAYOUTS)
def test_tile_multiples(cuda, layout, ta, tb):
    rng = np.random.default_rng(1)
    run_tc(cuda, rng, layout, ta, tb, 256, 128, 64, 1.0, 0.0)
    run_tc(cuda, rng, layout, ta, tb, 512, 768, 256, 1.0, 0.0)
    run_tc(cuda, rng, layout, ta, tb, 1024, 1024, 1024, 0.5, 0.0)


@pytest.mark.parametrize("layout,ta,tb", TC_LAYOUTS)
def test_ragged_edges_and_k_tail(cuda, layout, ta, tb):
    # m, n not multiples of the tile, k not a multiple of 64: TMA zero-fills, the epilogue masks
    rng = np.random.default_rng(2)
    run_tc(cuda, rng, layout, ta, tb, 200, 136, 72, 1.0, 0.0)
    run_tc(cuda, rng, layout, ta, tb, 336, 520, 200, 1.5, 0.0, pad=(8, 16, 3))
    run_tc(cuda, rng, layout, ta, tb, 1000, 1112, 1000, 1.0, 0.0, offs=(8, 16, 5), pad=(0, 8, 1))


@pytest.mark.parametrize("layout,ta,tb", TC_LAYOUTS)
def test_alpha_beta_epilogue(cuda, layout, ta, tb):
    rng = np.random.default_rng(3)
    run_tc(cuda, rng, layout, ta, tb, 384, 256, 128, 3.14, 3.14)
    run_tc(cuda, rng, layout, ta, tb, 640, 520, 320, 0.0, 1.0, pad=(8, 8, 8))
    run_tc(cuda, rng, layout, ta, tb, 304, 272, 136, -0.5, 0.25, offs=(24, 8, 7))


def test_many_tiles_per_cta_exercises_both_accumulators_and_the_ring(cuda):
    # 4096 x 3072: 24 x 16 = 384 tiles on 148 CTAs, so every CTA walks several tiles
    rng = np.random.default_rng(4)
    run_tc(cuda, rng, H.ROW, H.NO, H.YES, 3072, 4096, 512, 1.0, 0.0)


@pytest.mark.parametrize("layout,ta,tb", TC_LAYOUTS)
def test_cta_pair_kernel_and_single_cta_kernel_share_the_work(cuda, layout, ta, tb):
    """Problems with at least 256 rows (after layout normalisation) run on CTA pairs (two SMs per 256 x 256 tile);
    narrower ones, and small ones whose last pair tile would be half empty, keep one CTA per 128 x 256 tile."""
    rng = np.random.default_rng(6)
    swap = layout == H.ROW  # row-major problems are computed as the transposed column-major problem
    run_tc(cuda, rng, layout, ta, tb, *((136, 200) if swap else (200, 136)), 328, 1.0, 0.0)
    assert cb.last_kernel() == "tc_f16_128x256x64"
    run_tc(cuda, rng, layout, ta, tb, *((400, 336) if swap else (336, 400)), 328, 1.0, 0.5)
    assert cb.last_kernel() == "tc_f16_128x256x64"
    # ragged pair tiles: the second CTA of the last pair row holds 8 valid rows, the last column tile 72 columns
    run_tc(cuda, rng, layout, ta, tb, *((2120, 2184) if swap else (2184, 2120)), 520, -1.5, 0.5, offs=(8, 16, 3),
           pad=(8, 0, 5))
    assert cb.last_kernel() == "tc_f16_pair_256x256x64"
    # more tiles than CTA pairs: every pair walks several tiles, both accumulators and the whole ring are reused
    run_tc(cuda, rng, layout, ta, tb, 3072, 4096, 200, 1.0, 0.0)
    assert cb.last_kernel() == "tc_f16_pair_256x256x64"


def test_unaligned_operands_fall_back_to_the_cuda_core_kernel(cuda):
    rng = np.random.default_rng(5)
    run_tc(cuda, rng, H.ROW, H.NO, H.YES, 256, 256, 128, 1.0, 0.0, pad=(1, 0, 0), expect_tc=False)   # lda % 8 != 0
    run_tc(cuda, rng, H.ROW, H.NO, H.YES, 256, 256, 128, 1.0, 0.0, offs=(3, 0, 0), expect_tc=False)  # base not 16B


def test_config3_hgemm_8192_sampled(cuda):
    """The headline shape: 4096 sampled entries against exact fp64 dot products, and alpha-linearity
    (alpha = 2 doubles every result bit for bit)."""
    torch = cuda
    for m, n, k in ((8192, 8192, 8192), (16384, 4096, 8192)):
        g = torch.Generator(device="cuda").manual_seed(m)
        a = (torch.randn(m * k, generator=g, device="cuda") * 0.1).half()
        b = (torch.randn(n * k, generator=g, device="cuda") * 0.1).half()
        c1 = torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16)
        c2 = torch.full((m * n,), float("nan"), device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        assert cb.Gemm(H.ROW, H.NO, H.YES, m, n, k, 1.0, a, 0, k, b, 0, k, 0.0, c1, 0, n) == 0
        assert cb.last_kernel().startswith("tc_")
        assert cb.Gemm(H.ROW, H.NO, H.YES, m, n, k, 2.0, a, 0, k, b, 0, k, 0.0, c2, 0, n) == 0
        normal = c1.abs() >= 2.0 ** -13  # doubling is exact except for results in half's subnormal range
        assert torch.equal(c2[normal], c1[normal] * 2) and int(normal.sum()) > 0.99 * m * n
        rs = np.random.default_rng(m)
        rows, cols = rs.integers(0, m, 4096), rs.integers(0, n, 4096)
        want, mag = oracle.gemm_f64_sampled(16, H.ROW, H.NO, H.YES, k, 1.0, a.cpu().numpy(), 0, k, b.cpu().numpy(), 0, k,
                                            rows, cols)
        got = c1.cpu().numpy()[rows * n + cols].astype(np.float64)
        bad, worst = oracle.count_mismatches(16, got, want)
        assert bad == 0
        assert (np.abs(got - want) / mag).max() < 1e-4
        del a, b, c1, c2
