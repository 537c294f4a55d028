"""Parity of clblast::Gemm on the GPU (through the C ABI) against the CPU oracle.

Case grids follow the reference's own test strategy (test/correctness/testblas.hpp:138,506-594): sizes {7, 64},
both layouts, all transposes, offsets {0, 10}, alpha/beta from {0, 1, 3.14}, canary elements after each buffer.
Tolerances are the reference's own margins (test/correctness/tester.cpp:29-69) applied against the fp64 oracle:
fp32/fp64/complex: relative 5e-3 or absolute 1e-3; fp16: relative 8e-2 or absolute 0.15. A tighter normalised bound
|x - r| / sum_k|a||b| is asserted in addition (2^-20 for fp32, 2^-48 for fp64, 2e-3 for fp16 outputs).
"""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu

ALL_PRECISIONS = (32, 64, 16, 3232, 6464)
TIGHT = {32: 2.0 ** -20, 64: 2.0 ** -48, 16: 2e-3, 3232: 2.0 ** -19, 6464: 2.0 ** -47}


def transposes(precision):
    return (H.NO, H.YES, H.CONJ) if precision in (3232, 6464) else (H.NO, H.YES)


def run_and_check(torch, rng, precision, layout, ta, tb, m, n, k, alpha, beta, a_off=0, b_off=0, c_off=0,
                  ld_pad=(0, 0, 0), poison_c=False, expect_kernel=None, reject_kernel=None):
    case = H.gemm_case(rng, precision, layout, ta, tb, m, n, k, a_off, b_off, c_off, ld_pad, poison_c=poison_c)
    da, db, dc = (H.to_device(torch, precision, case[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.Gemm(layout, ta, tb, m, n, k, alpha, da, a_off, case["a_ld"], db, b_off, case["b_ld"], beta, dc, c_off,
                 case["c_ld"], precision=precision)
    assert st == cb.StatusCode.kSuccess, st
    if expect_kernel:
        assert expect_kernel in cb.last_kernel(), cb.last_kernel()
    if reject_kernel:
        assert reject_kernel not in cb.last_kernel(), cb.last_kernel()
    got = H.to_host(precision, dc)
    c_in = case["c"].copy()
    if poison_c:
        c_in[:] = 0  # beta == 0: whatever C held must not matter
    want = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alpha, case["a"], a_off, case["a_ld"], case["b"], b_off,
                           case["b_ld"], beta, c_in, c_off, case["c_ld"])
    mask = H.c_mask(layout, m, n, c_off, case["c_ld"], case["c"].size)
    H.check_against_oracle(precision, got, want, mask, case["c"])
    # normalised error: data is U[-2,2], so sum_k|a||b| <= 4k (8k for complex) and |beta*c| <= 2|beta|
    scale = (8.0 if precision > 100 else 4.0) * k * abs(alpha) + 2.0 * abs(beta) + 1e-30
    err = np.abs(H.oracle.widen(precision, got[mask]) - want[mask]).max() / scale
    assert err < TIGHT[precision], f"normalised error {err:.3e}"
    if precision in (32, 64) and cb.last_kernel().startswith("simt_"):
        # same order of operations as the reference kernels (k ascending, fused multiply-add, fused epilogue):
        # bit-identical to the reference-order oracle, which is itself bit-identical to the reference's kernel source
        typed = c_in.copy()
        oracle.gemm(precision, layout, ta, tb, m, n, k, alpha, case["a"], a_off, case["a_ld"], case["b"], b_off,
                    case["b_ld"], beta, typed, c_off, case["c_ld"])
        assert np.array_equal(got[mask].view(np.uint8), typed[mask].view(np.uint8)), "not bit-identical to the oracle"
    return err


@pytest.mark.parametrize("precision", ALL_PRECISIONS)
def test_reference_grid(cuda, precision):
    rng = np.random.default_rng(42)
    count = 0
    for layout, ta, tb in itertools.product((H.ROW, H.COL), transposes(precision), transposes(precision)):
        for m, n, k in itertools.product((7, 64), repeat=3):
            for off, pad in ((0, (0, 0, 0)), (10, (3, 1, 2))):
                alpha, beta = ((3.14, 3.14), (1.0, 0.0), (0.0, 1.0))[count % 3]
                if precision > 100:
                    alpha, beta = alpha + 0.5j, beta - 0.25j
                run_and_check(cuda, rng, precision, layout, ta, tb, m, n, k, alpha, beta, off, off, off, pad)
                count += 1
    assert count >= 128


@pytest.mark.parametrize("precision", ALL_PRECISIONS)
def test_ragged_shapes_hit_every_tile_class(cuda, precision):
    rng = np.random.default_rng(7)
    shapes = [(1, 1, 1), (1, 300, 17), (300, 1, 17), (17, 31, 129), (65, 127, 33), (130, 257, 70), (200, 96, 300),
              (1500, 1300, 70), (1409, 1537, 33), (64, 2000, 40), (2000, 64, 40), (60, 60, 100)]
    seen = set()
    for (m, n, k), (layout, ta, tb) in zip(shapes * 2, itertools.cycle(
            itertools.product((H.COL, H.ROW), transposes(precision), transposes(precision)))):
        run_and_check(cuda, rng, precision, layout, ta, tb, m, n, k, 1.5, 0.5, 3, 5, 7, (5, 1, 3))
        seen.add(cb.last_kernel().rsplit("_", 1)[-1])
    assert {"32x32", "64x64"} <= seen
    if precision < 100:
        assert {"128x128", "64x128"} <= seen


@pytest.mark.parametrize("precision", (32, 64, 16))
def test_aligned_fast_paths_all_transposes(cuda, precision):
    # aligned pointers and leading dimensions take the 16-byte load/store paths of every kernel variant
    rng = np.random.default_rng(11)
    for layout, ta, tb in itertools.product((H.ROW, H.COL), (H.NO, H.YES), (H.NO, H.YES)):
        run_and_check(cuda, rng, precision, layout, ta, tb, 1536, 1280, 256, 1.5, 0.5)
        run_and_check(cuda, rng, precision, layout, ta, tb, 256, 192, 128, 0.7, 0.3, 16, 32, 64, (16, 32, 8))


@pytest.mark.parametrize("precision", ALL_PRECISIONS)
def test_beta_zero_never_reads_c(cuda, precision):
    rng = np.random.default_rng(3)
    for m, n, k in ((64, 64, 64), (7, 64, 7), (300, 200, 100), (1500, 1300, 40)):
        run_and_check(cuda, rng, precision, H.COL, H.NO, H.YES, m, n, k, 1.0, 0.0, poison_c=True)
        run_and_check(cuda, rng, precision, H.ROW, H.NO, H.NO, m, n, k, 1.0, 0.0, 1, 2, 3, (1, 1, 1), poison_c=True)


def test_config1_sgemm_1024_row_major(cuda):
    # SGEMM 1024^3, row-major NN, alpha 0.7, beta 0.3, U[-1,1]
    rng = np.random.default_rng(1)
    n = 1024
    a = rng.uniform(-1, 1, n * n).astype(np.float32)
    b = rng.uniform(-1, 1, n * n).astype(np.float32)
    c = rng.uniform(-1, 1, n * n).astype(np.float32)
    da, db, dc = (cuda.from_numpy(x).cuda() for x in (a, b, c))
    cuda.cuda.synchronize()
    assert cb.Gemm(H.ROW, H.NO, H.NO, n, n, n, 0.7, da, 0, n, db, 0, n, 0.3, dc, 0, n) == cb.StatusCode.kSuccess
    got = dc.cpu().numpy().astype(np.float64)
    want = 0.7 * (a.reshape(n, n).astype(np.float64) @ b.reshape(n, n).astype(np.float64)) + 0.3 * c.reshape(n, n)
    bad, worst = oracle.count_mismatches(32, got.ravel(), want.ravel())
    assert bad == 0
    assert worst / (0.7 * n + 0.3) < 2.0 ** -21
    # and against the reference-order fp32 oracle: same order of operations, so bit-identical
    c_ref = c.copy()
    oracle.gemm(32, H.ROW, H.NO, H.NO, n, n, n, 0.7, a, 0, n, b, 0, n, 0.3, c_ref, 0, n)
    if cb.last_kernel().startswith("tc_"):   # 3xTF32 tensor-core path: fp32-level accuracy, not the same bits
        assert np.abs(dc.cpu().numpy().astype(np.float64) - c_ref).max() / (0.7 * n + 0.3) < 2.0 ** -21
    else:
        assert np.array_equal(dc.cpu().numpy().view(np.uint8), c_ref.view(np.uint8))


@pytest.mark.parametrize("n", (256, 512, 1000))
def test_config2_sgemm_sweep_col_major(cuda, n):
    rng = np.random.default_rng(n)
    for ta, tb in itertools.product((H.NO, H.YES), repeat=2):
        case = H.gemm_case(rng, 32, H.COL, ta, tb, n, n, n, ld_pad=(16, 16, 16), lo=-1, hi=1)
        for key in "abc":  # padding between columns holds NaN canaries
            buf = case[key]
            ld = case[key + "_ld"]
            view = buf[: (buf.size - H.CANARY) // ld * ld].reshape(-1, ld)
            view[:, n:] = np.nan
        da, db, dc = (H.to_device(cuda, 32, case[x]) for x in "abc")
        cuda.cuda.synchronize()
        st = cb.Gemm(H.COL, ta, tb, n, n, n, 1.5, da, 0, case["a_ld"], db, 0, case["b_ld"], 0.5, dc, 0, case["c_ld"])
        assert st == cb.StatusCode.kSuccess
        got = dc.cpu().numpy()
        want = oracle.gemm_f64(32, H.COL, ta, tb, n, n, n, 1.5, case["a"], 0, case["a_ld"], case["b"], 0, case["b_ld"],
                               0.5, case["c"], 0, case["c_ld"])
        mask = H.c_mask(H.COL, n, n, 0, case["c_ld"], case["c"].size)
        worst = H.check_against_oracle(32, got, want, mask, case["c"])
        assert worst / (1.5 * n + 0.5) < 2.0 ** -21


def test_config2_ragged_unaligned_leading_dimensions(cuda):
    rng = np.random.default_rng(5)
    m, n, k = 4097, 3071, 1025
    for ta, tb in itertools.product((H.NO, H.YES), repeat=2):
        case = H.gemm_case(rng, 32, H.COL, ta, tb, m, n, k, ld_pad=(16, 16, 16), lo=-1, hi=1)
        da, db, dc = (H.to_device(cuda, 32, case[x]) for x in "abc")
        cuda.cuda.synchronize()
        st = cb.Gemm(H.COL, ta, tb, m, n, k, 1.5, da, 0, case["a_ld"], db, 0, case["b_ld"], 0.5, dc, 0, case["c_ld"])
        assert st == cb.StatusCode.kSuccess
        got = dc.cpu().numpy()
        want = oracle.gemm_f64(32, H.COL, ta, tb, m, n, k, 1.5, case["a"], 0, case["a_ld"], case["b"], 0, case["b_ld"],
                               0.5, case["c"], 0, case["c_ld"])
        mask = H.c_mask(H.COL, m, n, 0, case["c_ld"], case["c"].size)
        worst = H.check_against_oracle(32, got, want, mask, case["c"])
        assert worst / (1.5 * k + 0.5) < 2.0 ** -21


@pytest.mark.parametrize("precision,n", ((32, 4096), (32, 8192), (64, 4096)))
def test_large_square_sampled(cuda, precision, n):
    """Full-size cases are checked on 4096 sampled entries, each an exact fp64 dot product of length K, plus a
    linearity property: gemm(alpha=2) == 2 * gemm(alpha=1) bit for bit (scaling by 2 is exact)."""
    torch = cuda
    dt = getattr(torch, H.TORCH_NAME[precision])
    g = torch.Generator(device="cuda").manual_seed(n)
    a = (torch.rand(n * n, generator=g, device="cuda", dtype=dt) * 2 - 1)
    b = (torch.rand(n * n, generator=g, device="cuda", dtype=dt) * 2 - 1)
    c1 = torch.full((n * n,), float("nan"), device="cuda", dtype=dt)
    c2 = torch.full((n * n,), float("nan"), device="cuda", dtype=dt)
    torch.cuda.synchronize()
    for ta, tb in ((H.NO, H.NO), (H.YES, H.NO)):
        assert cb.Gemm(H.COL, ta, tb, n, n, n, 1.0, a, 0, n, b, 0, n, 0.0, c1, 0, n) == cb.StatusCode.kSuccess
        assert cb.Gemm(H.COL, ta, tb, n, n, n, 2.0, a, 0, n, b, 0, n, 0.0, c2, 0, n) == cb.StatusCode.kSuccess
        assert torch.equal(c2, c1 * 2)
        rs = np.random.default_rng(n)
        rows = rs.integers(0, n, 4096)
        cols = rs.integers(0, n, 4096)
        ah, bh = a.cpu().numpy(), b.cpu().numpy()
        want, mag = oracle.gemm_f64_sampled(precision, H.COL, ta, tb, n, 1.0, ah, 0, n, bh, 0, n, rows, cols)
        got = c1.cpu().numpy()[cols * n + rows].astype(np.float64)
        bad, _ = oracle.count_mismatches(precision, got, want)
        assert bad == 0
        assert (np.abs(got - want) / mag).max() < TIGHT[precision]


def test_forcing_the_small_tile_family_through_override_parameters(cuda):
    # the reference's tests force its direct kernels with XGEMM_MIN_INDIRECT_SIZE (test/routines/level3/xgemm.hpp:62-70)
    rng = np.random.default_rng(9)
    dev = cuda.cuda.current_device()
    try:
        assert cb.OverrideParameters(dev, "GemmRoutine", 32, {"XGEMM_MIN_INDIRECT_SIZE": 4096}) == 0
        run_and_check(cuda, rng, 32, H.COL, H.NO, H.NO, 300, 200, 100, 1.5, 0.5, expect_kernel="32x32")
        assert cb.OverrideParameters(dev, "GemmRoutine", 32, {"XGEMM_MIN_INDIRECT_SIZE": 0}) == 0
        run_and_check(cuda, rng, 32, H.COL, H.NO, H.NO, 300, 200, 100, 1.5, 0.5, reject_kernel="32x32")
    finally:
        cb.OverrideParameters(dev, "GemmRoutine", 32, {"XGEMM_MIN_INDIRECT_SIZE": 0})


def test_async_call_on_a_caller_stream(cuda):
    torch = cuda
    rng = np.random.default_rng(2)
    n = 512
    a = torch.from_numpy(rng.uniform(-1, 1, n * n).astype(np.float32)).cuda()
    b = torch.from_numpy(rng.uniform(-1, 1, n * n).astype(np.float32)).cuda()
    c = torch.zeros(n * n, device="cuda")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    before = cb.launch_count()
    with torch.cuda.stream(s):
        assert cb.Gemm(H.COL, H.NO, H.NO, n, n, n, 1.0, a, 0, n, b, 0, n, 0.0, c, 0, n, stream=s) == 0
    s.synchronize()
    assert cb.launch_count() == before + 1
    want = (b.view(n, n).double() @ a.view(n, n).double())  # column-major data seen as row-major transposes
    assert torch.allclose(c.view(n, n).double(), want, atol=1e-3)
