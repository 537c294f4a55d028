"""Batched calls with problems large enough for the tensor cores: GemmStridedBatched, and GemmBatched whose offset
tables are evenly spaced, address the whole batch through one three-dimensional tensor map per operand. Checked
against a loop of fp64 oracle GEMMs, as the reference's own tests define the batched routines
(test/routines/levelx/xgemmstridedbatched.hpp:131-141, xgemmbatched.hpp:154-162)."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H
from tests.test_batched_gpu import strided_case

pytestmark = pytest.mark.gpu

LAYOUTS = list(itertools.product((H.COL, H.ROW), (H.NO, H.YES), (H.NO, H.YES)))


def check(torch, precision, layout, ta, tb, m, n, k, batch, alphas, betas, g, a_offs, b_offs, c_offs, got):
    """Every problem of the batch against the fp64 oracle; everything outside the results untouched."""
    want = oracle.widen(precision, g["c"])
    mask = np.zeros(g["c"].size, dtype=bool)
    for i in range(batch):
        out = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alphas[i], g["a"], a_offs[i], g["a_ld"], g["b"],
                              b_offs[i], g["b_ld"], betas[i], g["c"], c_offs[i], g["c_ld"])
        one = H.c_mask(layout, m, n, c_offs[i], g["c_ld"], g["c"].size)
        want[one] = out[one]
        mask |= one
    worst = H.check_against_oracle(precision, got, want, mask, g["c"])
    bound = (2.0 ** -20 if precision == 32 else 1e-3) * (max(abs(x) for x in alphas) * k + max(abs(x) for x in betas))
    assert worst <= bound + 1e-6, (worst, bound)


def run_strided(torch, rng, precision, layout, ta, tb, m, n, k, batch, alpha, beta, pad, off, expect):
    g = strided_case(rng, precision, layout, ta, tb, m, n, k, batch, pad, off, -1.0, 1.0)
    da, db, dc = (H.to_device(torch, precision, g[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.GemmStridedBatched(layout, ta, tb, m, n, k, alpha, da, off, g["a_ld"], g["a_stride"], db, off, g["b_ld"],
                               g["b_stride"], beta, dc, off, g["c_ld"], g["c_stride"], batch, precision=precision)
    assert st == cb.StatusCode.kSuccess, st
    assert cb.last_kernel().startswith(expect), cb.last_kernel()
    offs = lambda key: [off + i * g[key + "_stride"] for i in range(batch)]
    check(torch, precision, layout, ta, tb, m, n, k, batch, [alpha] * batch, [beta] * batch, g, offs("a"), offs("b"),
          offs("c"), H.to_host(precision, dc))


@pytest.mark.parametrize("layout,ta,tb", LAYOUTS)
def test_strided_batched_hgemm(cuda, layout, ta, tb):
    rng = np.random.default_rng(1)
    # 12 problems of 512 x 512: two SMs per 256 x 256 tile; ragged 200-row problems: one CTA per tile
    run_strided(cuda, rng, 16, layout, ta, tb, 512, 512, 136, 12, 1.5, 0.5, 8, 16, "tc_f16_pair")
    swap = layout == H.ROW
    run_strided(cuda, rng, 16, layout, ta, tb, *((328, 200) if swap else (200, 328)), 72, 5, 1.0, 0.0, 8, 0,
                "tc_f16_128x256x64")


@pytest.mark.parametrize("layout,ta,tb", LAYOUTS)
def test_strided_batched_sgemm(cuda, layout, ta, tb):
    rng = np.random.default_rng(2)
    run_strided(cuda, rng, 32, layout, ta, tb, 520, 392, 136, 9, 1.5, 0.5, 4, 8, "tc_f32_3xtf32_128x128x32")
    # leading dimensions and strides that are not multiples of four elements: gathered operands
    run_strided(cuda, rng, 32, layout, ta, tb, 520, 392, 136, 9, -1.0, 0.0, 3, 5, "tc_f32_3xtf32_gather")
    # few tiles in the whole batch: every tile of every problem is split along K over a cluster of two CTAs
    run_strided(cuda, rng, 32, layout, ta, tb, 520, 392, 296, 3, 0.75, -0.5, 4, 8, "tc_f32_3xtf32_128x128x32_splitk2")


def test_strided_batched_sgemm_on_cta_pairs(cuda):
    rng = np.random.default_rng(3)
    # 40 problems of 512 x 512: 160 tiles of 256 x 256
    run_strided(cuda, rng, 32, H.COL, H.NO, H.YES, 512, 512, 160, 40, 1.0, 1.0, 4, 4, "tc_f32_3xtf32_pair")


@pytest.mark.parametrize("precision,expect", ((16, "tc_f16_pair"), (32, "tc_f32_3xtf32")))
def test_shared_operand_has_stride_zero(cuda, precision, expect):
    """One B for all problems (stride 0), as in a batch of activations times one weight matrix."""
    torch = cuda
    rng = np.random.default_rng(4)
    m, n, k, batch = 512, 384, 128, 6
    g = strided_case(rng, precision, H.COL, H.NO, H.NO, m, n, k, batch, 8, 0, -1.0, 1.0)
    da, db, dc = (H.to_device(torch, precision, g[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.GemmStridedBatched(H.COL, H.NO, H.NO, m, n, k, 1.0, da, 0, g["a_ld"], g["a_stride"], db, 0, g["b_ld"], 0,
                               0.0, dc, 0, g["c_ld"], g["c_stride"], batch, precision=precision)
    assert st == cb.StatusCode.kSuccess, st
    assert cb.last_kernel().startswith(expect), cb.last_kernel()
    check(torch, precision, H.COL, H.NO, H.NO, m, n, k, batch, [1.0] * batch, [0.0] * batch, g,
          [i * g["a_stride"] for i in range(batch)], [0] * batch, [i * g["c_stride"] for i in range(batch)],
          H.to_host(precision, dc))


@pytest.mark.parametrize("precision,expect", ((16, "tc_f16"), (32, "tc_f32")))
@pytest.mark.parametrize("layout", (H.COL, H.ROW))
def test_offset_table_batches(cuda, precision, expect, layout):
    """GemmBatched: evenly spaced offsets with per-problem alpha and beta run on the tensor cores; a permuted table
    (not expressible with strides) and a table of one entry with a non-zero offset stay correct."""
    torch = cuda
    rng = np.random.default_rng(5)
    m, n, k, batch = 384, 512, 136, 7
    g = strided_case(rng, precision, layout, H.NO, H.YES, m, n, k, batch, 8, 16, -1.0, 1.0)
    alphas = [1.0 + 0.25 * i for i in range(batch)]
    betas = [0.0 if i % 2 else 0.5 for i in range(batch)]
    offs = {key: [16 + i * g[key + "_stride"] for i in range(batch)] for key in "abc"}

    def call(a_offs, b_offs, c_offs, count):
        da, db, dc = (H.to_device(torch, precision, g[x]) for x in "abc")
        torch.cuda.synchronize()
        st = cb.GemmBatched(layout, H.NO, H.YES, m, n, k, alphas[:count], da, a_offs, g["a_ld"], db, b_offs, g["b_ld"],
                            betas[:count], dc, c_offs, g["c_ld"], count, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        check(torch, precision, layout, H.NO, H.YES, m, n, k, count, alphas, betas, g, a_offs, b_offs, c_offs,
              H.to_host(precision, dc))
        return cb.last_kernel()

    assert call(offs["a"], offs["b"], offs["c"], batch).startswith(expect)
    order = list(rng.permutation(batch))
    permuted = call([offs["a"][j] for j in order], offs["b"], offs["c"], batch)
    assert permuted.startswith("simt_"), permuted
    single = call(offs["a"][3:4], offs["b"][2:3], offs["c"][5:6], 1)
    assert single.startswith(expect if precision == 16 else "tc_f32_3xtf32"), single


@pytest.mark.parametrize("layout,ta,tb", LAYOUTS)
def test_narrow_problems_run_transposed_on_the_tensor_cores(cuda, layout, ta, tb):
    """Batches whose problems have at most 64 rows of C (after layout normalisation) and at least 64 columns: the
    kernel computes C^T = op(B)^T op(A)^T, so the narrow extent becomes the MMA's N. Ragged extents, K tail, a
    leading dimension of C that rules out 16-byte stores, beta from zero and non-zero."""
    rng = np.random.default_rng(8)
    swap = layout == H.ROW
    shape = lambda narrow, wide: (wide, narrow) if swap else (narrow, wide)
    run_strided(cuda, rng, 32, layout, ta, tb, *shape(64, 128), 96, 300, 1.0, 1.0, 0, 0, "tc_f32_3xtf32_narrow")
    run_strided(cuda, rng, 32, layout, ta, tb, *shape(48, 200), 72, 240, -1.5, 0.5, 4, 8, "tc_f32_3xtf32_narrow")
    run_strided(cuda, rng, 32, layout, ta, tb, *shape(20, 136), 100, 600, 2.0, 0.0, 4, 4, "tc_f32_3xtf32_narrow")


def test_narrow_problems_with_offset_tables_and_odd_c_stride(cuda):
    torch = cuda
    rng = np.random.default_rng(9)
    m, n, k, batch = 64, 128, 96, 320
    g = strided_case(rng, 32, H.COL, H.NO, H.NO, m, n, k, batch, 4, 0, -1.0, 1.0)
    g["c_ld"] = m + 1   # C needs no alignment: scalar stores
    g["c_stride"] = g["c_ld"] * n + 3
    g["c"] = H.rand_buffer(rng, 32, 5 + g["c_stride"] * batch + H.CANARY, -1.0, 1.0)
    alphas = [1.0 + 0.01 * i for i in range(batch)]
    betas = [0.0 if i % 3 else 0.5 for i in range(batch)]
    a_offs = [i * g["a_stride"] for i in range(batch)]
    b_offs = [i * g["b_stride"] for i in range(batch)]
    c_offs = [5 + i * g["c_stride"] for i in range(batch)]
    da, db, dc = (H.to_device(torch, 32, g[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.GemmBatched(H.COL, H.NO, H.NO, m, n, k, alphas, da, a_offs, g["a_ld"], db, b_offs, g["b_ld"], betas, dc,
                        c_offs, g["c_ld"], batch, precision=32)
    assert st == cb.StatusCode.kSuccess, st
    assert cb.last_kernel().startswith("tc_f32_3xtf32_narrow"), cb.last_kernel()
    check(torch, 32, H.COL, H.NO, H.NO, m, n, k, batch, alphas, betas, g, a_offs, b_offs, c_offs, H.to_host(32, dc))
