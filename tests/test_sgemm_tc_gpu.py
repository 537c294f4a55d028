"""The tensor-core SGEMM kernel (error-compensated 3xTF32 on tcgen05) against the fp64 oracle.

Tolerance: the reference's fp32 margins (relative 5e-3 or absolute 1e-3, test/correctness/tester.cpp:29-69) and the
fp32-quality bound |x - r| <= 2^-20 * (|alpha| * sum_k|a||b| + |beta||c|); the kernel is not bit-identical to the
k-ascending reference order, the CUDA-core kernel (B200BLAS_SGEMM=ffma, or any smaller problem) is."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu


def run_tc32(torch, rng, layout, ta, tb, m, n, k, alpha, beta, offs=(0, 0, 0), pad=(0, 0, 0), expect_tc=True):
    case = H.gemm_case(rng, 32, layout, ta, tb, m, n, k, offs[0], offs[1], offs[2], pad, lo=-1, hi=1,
                       poison_c=(beta == 0))
    da, db, dc = (H.to_device(torch, 32, case[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.Gemm(layout, ta, tb, m, n, k, alpha, da, offs[0], case["a_ld"], db, offs[1], case["b_ld"], beta, dc, offs[2],
                 case["c_ld"], precision=32)
    assert st == cb.StatusCode.kSuccess, st
    assert cb.last_kernel().startswith("tc_f32") == expect_tc, cb.last_kernel()
    got = H.to_host(32, dc)
    c_in = case["c"].copy()
    if beta == 0:
        c_in[:] = 0
    want = oracle.gemm_f64(32, layout, ta, tb, m, n, k, alpha, case["a"], offs[0], case["a_ld"], case["b"], offs[1],
                           case["b_ld"], beta, c_in, offs[2], case["c_ld"])
    mask = H.c_mask(layout, m, n, offs[2], case["c_ld"], case["c"].size)
    worst = H.check_against_oracle(32, got, want, mask, case["c"])
    # data is U[-1,1]: sum_k|a||b| <= k
    assert worst <= 2.0 ** -20 * (abs(alpha) * k + abs(beta)), worst / (abs(alpha) * k + abs(beta))
    return worst


ALL = list(itertools.product((H.COL, H.ROW), (H.NO, H.YES), (H.NO, H.YES)))


@pytest.mark.parametrize("layout,ta,tb", ALL)
def test_all_operand_orientations(cuda, layout, ta, tb):
    rng = np.random.default_rng(1)
    run_tc32(cuda, rng, layout, ta, tb, 512, 512, 512, 1.0, 0.0)
    run_tc32(cuda, rng, layout, ta, tb, 768, 1024, 256, 1.5, 0.5)


@pytest.mark.parametrize("layout,ta,tb", ALL)
def test_ragged_edges_k_tail_offsets(cuda, layout, ta, tb):
    rng = np.random.default_rng(2)
    run_tc32(cuda, rng, layout, ta, tb, 1000, 1112, 520, 1.5, 0.5, offs=(4, 8, 3), pad=(4, 8, 1))
    run_tc32(cuda, rng, layout, ta, tb, 700, 900, 300, -0.5, 0.0, pad=(12, 0, 5))


@pytest.mark.parametrize("layout,ta,tb", ALL)
def test_cta_pair_kernel_ragged(cuda, layout, ta, tb):
    """At least 148 tiles of 256 x 256: two SMs share a tile (cta_group::2). Ragged M / N / K, offsets, padded leading
    dimensions, alpha and beta."""
    rng = np.random.default_rng(7)
    run_tc32(cuda, rng, layout, ta, tb, 3080, 3332, 168, 1.5, 0.5, offs=(4, 8, 3), pad=(4, 8, 1))
    assert cb.last_kernel() == "tc_f32_3xtf32_pair_256x256x32"


def test_small_problems_keep_the_cuda_core_kernel(cuda):
    rng = np.random.default_rng(3)
    run_tc32(cuda, rng, H.COL, H.NO, H.NO, 200, 200, 200, 1.0, 0.0, expect_tc=False)
    run_tc32(cuda, rng, H.COL, H.NO, H.NO, 200, 200, 200, 1.0, 0.0, pad=(1, 0, 0), expect_tc=False)


@pytest.mark.parametrize("layout,ta,tb", ALL)
def test_unaligned_operands_are_gathered_on_the_tensor_cores(cuda, layout, ta, tb):
    """Leading dimensions that are not multiples of four elements, or bases off the 16-byte grid, cannot travel by
    TMA: the split warps load such operands with bounds-checked scalar loads instead. Every orientation, odd
    leading dimensions, odd offsets, ragged M / N / K."""
    rng = np.random.default_rng(4)
    run_tc32(cuda, rng, layout, ta, tb, 600, 600, 600, 1.0, 0.0, pad=(1, 0, 0))     # lda % 4 != 0
    assert cb.last_kernel().startswith("tc_f32_3xtf32_gather")
    run_tc32(cuda, rng, layout, ta, tb, 600, 600, 600, 1.0, 0.0, offs=(2, 0, 0))    # base of A not 16-byte aligned
    assert cb.last_kernel().startswith("tc_f32_3xtf32_gather")
    run_tc32(cuda, rng, layout, ta, tb, 1001, 777, 515, -1.25, 0.75, offs=(3, 5, 7), pad=(3, 1, 2))
    assert cb.last_kernel().startswith("tc_f32_3xtf32_gather")
    run_tc32(cuda, rng, layout, ta, tb, 513, 1025, 300, 1.0, 0.0, offs=(0, 1, 0), pad=(0, 0, 0))
    assert cb.last_kernel().startswith("tc_f32_3xtf32_gather")


def test_config2_ragged_shape(cuda):
    """4097 x 3071 x 1025 with leading dimensions 16 past the extents: sampled against the fp64 oracle."""
    torch = cuda
    m, n, k = 4097, 3071, 1025
    g = torch.Generator(device="cuda").manual_seed(5)
    rs = np.random.default_rng(5)
    for ta, tb in itertools.product((H.NO, H.YES), repeat=2):
        a_rows, a_cols = (m, k) if ta == H.NO else (k, m)
        b_rows, b_cols = (k, n) if tb == H.NO else (n, k)
        lda, ldb, ldc = a_rows + 16, b_rows + 16, m + 16
        a = torch.rand(lda * a_cols, generator=g, device="cuda") * 2 - 1
        b = torch.rand(ldb * b_cols, generator=g, device="cuda") * 2 - 1
        c0 = torch.rand(ldc * n, generator=g, device="cuda") * 2 - 1
        c = c0.clone()
        torch.cuda.synchronize()
        assert cb.Gemm(H.COL, ta, tb, m, n, k, 1.5, a, 0, lda, b, 0, ldb, 0.5, c, 0, ldc) == 0
        assert cb.last_kernel().startswith(("tc_f32", "repitched_tc_f32")), cb.last_kernel()
        rows, cols = rs.integers(0, m, 2048), rs.integers(0, n, 2048)
        rows[:4], cols[:4] = (0, m - 1, 0, m - 1), (0, 0, n - 1, n - 1)
        ah, bh = a.cpu().numpy().astype(np.float64), b.cpu().numpy().astype(np.float64)
        # column-major storage read as [column][row]: op(A) as [m][k], op(B) as [n][k]
        opa = ah.reshape(a_cols, lda)[:, :a_rows]
        opa = opa.T if ta == H.NO else opa
        opb = bh.reshape(b_cols, ldb)[:, :b_rows]
        opb = opb if tb == H.NO else opb.T
        want = 1.5 * np.einsum("ik,ik->i", opa[rows], opb[cols]) + 0.5 * c0.cpu().numpy()[cols * ldc + rows]
        mag = 1.5 * np.einsum("ik,ik->i", np.abs(opa[rows]), np.abs(opb[cols])) + 0.5
        got = c.cpu().numpy()[cols * ldc + rows].astype(np.float64)
        assert (np.abs(got - want) / mag).max() < 2.0 ** -20
        assert torch.equal(c.view(n, ldc)[:, m:], c0.view(n, ldc)[:, m:])


def test_infinite_inputs_stay_confined_to_their_outputs(cuda):
    """An infinite operand makes exactly the outputs it touches non-finite (NaN or inf: the split arithmetic can turn
    inf into NaN, which the reference's comparison rule accepts as equal); everything else stays finite."""
    torch = cuda
    n = 512
    a = torch.rand(n * n, device="cuda") + 0.5
    b = torch.rand(n * n, device="cuda") + 0.5
    a[5] = float("inf")  # column-major A: element (5, 0)
    c = torch.zeros(n * n, device="cuda")
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, n, n, n, 1.0, a, 0, n, b, 0, n, 0.0, c, 0, n) == 0
    assert cb.last_kernel().startswith("tc_f32")
    finite = torch.isfinite(c.view(n, n))   # [j][i] holds C(i, j)
    assert not finite[:, 5].any()
    finite[:, 5] = True
    assert finite.all()


@pytest.mark.parametrize("n", (4096, 8192))
def test_config2_large_squares_sampled(cuda, n):
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(n)
    ld = n + 16
    a = torch.rand(ld * n, generator=g, device="cuda") * 2 - 1
    b = torch.rand(ld * n, generator=g, device="cuda") * 2 - 1
    c0 = torch.rand(ld * n, generator=g, device="cuda") * 2 - 1
    rs = np.random.default_rng(n)
    rows, cols = rs.integers(0, n, 4096), rs.integers(0, n, 4096)
    ah, bh, ch = a.cpu().numpy(), b.cpu().numpy(), c0.cpu().numpy()
    for ta, tb in itertools.product((H.NO, H.YES), repeat=2):
        c = c0.clone()
        torch.cuda.synchronize()
        assert cb.Gemm(H.COL, ta, tb, n, n, n, 1.5, a, 0, ld, b, 0, ld, 0.5, c, 0, ld) == 0
        assert cb.last_kernel().startswith("tc_f32")
        want, mag = oracle.gemm_f64_sampled(32, H.COL, ta, tb, n, 1.5, ah, 0, ld, bh, 0, ld, rows, cols)
        want = want + 0.5 * ch[cols * ld + rows].astype(np.float64)
        got = c.cpu().numpy()[cols * ld + rows].astype(np.float64)
        bad, _ = oracle.count_mismatches(32, got, want)
        assert bad == 0
        assert (np.abs(got - want) / (1.5 * mag + 0.5)).max() < 2.0 ** -20
        # the padding between columns is untouched
        assert torch.equal(c.view(n, ld)[:, n:], c0.view(n, ld)[:, n:])


@pytest.mark.parametrize("shift", (100, 120))
def test_wide_dynamic_range_operands(cuda, shift):
    """A scaled by 2^-shift, B by 2^+shift: every product is well scaled, so the fp32 FFMA chain of the reference gives
    fp32-level results. The split keeps that level as long as the small part x - tf32(x) (at most 2^-11 |x|) of the
    contributing entries is a normal fp32 number, i.e. for |x| >= 2^-115: asserted at 2^-100. Below that the small
    parts become subnormal and the guaranteed level is the TF32 one (2^-10 of sum |a||b|): pinned at 2^-120."""
    torch = cuda
    n = 512
    rng = np.random.default_rng(shift)
    a = (rng.uniform(-1, 1, n * n) * 2.0 ** -shift).astype(np.float32)
    b = (rng.uniform(-1, 1, n * n) * 2.0 ** shift).astype(np.float32)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.full((n * n,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, n, n, n, 1.0, da, 0, n, db, 0, n, 0.0, c, 0, n) == 0
    assert cb.last_kernel().startswith("tc_f32")
    want = b.astype(np.float64).reshape(n, n) @ a.astype(np.float64).reshape(n, n)   # [j][i] = C(i, j)
    mag = np.abs(b.astype(np.float64)).reshape(n, n) @ np.abs(a.astype(np.float64)).reshape(n, n)
    got = c.cpu().numpy().astype(np.float64).reshape(n, n)
    assert np.isfinite(got).all()
    err = (np.abs(got - want) / mag).max()
    assert err < (2.0 ** -20 if shift == 100 else 2.0 ** -9), err


def test_values_next_to_the_largest_finite_float(cuda):
    """Entries within the last 2^-11 of the fp32 range would round to infinity as TF32; the split saturates them
    instead, so a product that is finite in fp32 arithmetic stays finite and accurate."""
    torch = cuda
    n = 512
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, n * n).astype(np.float32)
    big = np.float32(3.4028234e38)
    a[::97] = big * np.where(rng.uniform(size=a[::97].size) < 0.5, -1, 1).astype(np.float32)
    b = (rng.uniform(-1, 1, n * n) * 2.0 ** -12).astype(np.float32)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.full((n * n,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, n, n, n, 1.0, da, 0, n, db, 0, n, 0.0, c, 0, n) == 0
    assert cb.last_kernel().startswith("tc_f32")
    want = b.astype(np.float64).reshape(n, n) @ a.astype(np.float64).reshape(n, n)
    mag = np.abs(b.astype(np.float64)).reshape(n, n) @ np.abs(a.astype(np.float64)).reshape(n, n)
    got = c.cpu().numpy().astype(np.float64).reshape(n, n)
    assert np.isfinite(got).all()
    assert (np.abs(got - want) / mag).max() < 2.0 ** -20


@pytest.mark.parametrize("precision", (32, 16))
def test_large_problems_with_unaligned_operands_are_repitched(cuda, precision):
    """Operands TMA cannot address (odd leading dimension, base off the 16-byte grid) of a large product are copied once
    into scratch with an aligned pitch and multiplied by the TMA kernels; every orientation, sampled against exact fp64
    dot products, padding between the columns of C untouched."""
    torch = cuda
    dt = torch.float32 if precision == 32 else torch.float16
    m, n, k = 2049, 1500, 520
    g = torch.Generator(device="cuda").manual_seed(11)
    rs = np.random.default_rng(11)
    for ta, tb in itertools.product((H.NO, H.YES), repeat=2):
        a_rows, a_cols = (m, k) if ta == H.NO else (k, m)
        b_rows, b_cols = (k, n) if tb == H.NO else (n, k)
        lda, ldb, ldc = a_rows + 3, b_rows + 1, m + 5
        a_off, b_off = 1, 2
        a = ((torch.rand(a_off + lda * a_cols, generator=g, device="cuda") * 2 - 1) * 0.5).to(dt)
        b = ((torch.rand(b_off + ldb * b_cols, generator=g, device="cuda") * 2 - 1) * 0.5).to(dt)
        c0 = (torch.rand(ldc * n, generator=g, device="cuda") * 2 - 1).to(dt)
        c = c0.clone()
        torch.cuda.synchronize()
        assert cb.Gemm(H.COL, ta, tb, m, n, k, 1.5, a, a_off, lda, b, b_off, ldb, 0.5, c, 0, ldc) == 0
        assert cb.last_kernel().startswith("repitched_tc_"), cb.last_kernel()
        rows, cols = rs.integers(0, m, 2048), rs.integers(0, n, 2048)
        rows[:4], cols[:4] = (0, m - 1, 0, m - 1), (0, 0, n - 1, n - 1)
        ah, bh = a[a_off:].cpu().numpy().astype(np.float64), b[b_off:].cpu().numpy().astype(np.float64)
        opa = ah.reshape(a_cols, lda)[:, :a_rows]
        opa = opa.T if ta == H.NO else opa
        opb = bh.reshape(b_cols, ldb)[:, :b_rows]
        opb = opb if tb == H.NO else opb.T
        old = c0.cpu().numpy().astype(np.float64)[cols * ldc + rows]
        want = 1.5 * np.einsum("ik,ik->i", opa[rows], opb[cols]) + 0.5 * old
        mag = 1.5 * np.einsum("ik,ik->i", np.abs(opa[rows]), np.abs(opb[cols])) + 0.5
        got = c.cpu().numpy().astype(np.float64)[cols * ldc + rows]
        assert (np.abs(got - want) / mag).max() < (2.0 ** -20 if precision == 32 else 2e-3)
        assert torch.equal(c.view(n, ldc)[:, m:], c0.view(n, ldc)[:, m:])


_VARIANT_SCRIPT = r"""
import hashlib, sys
import torch
import clblast_b200 as cb
ROW, COL, NO, YES = 101, 102, 111, 112
g = torch.Generator(device="cuda").manual_seed(5)
def rnd(n):
    return torch.rand(n, generator=g, device="cuda") * 2 - 1
out = []
# 128 x 64 tiles (few tiles), 128 x 128 tiles, a narrow batch, a convolution
for (layout, ta, tb, m, n, k) in ((ROW, NO, NO, 1024, 1024, 1024), (COL, YES, NO, 1536, 1280, 520), (COL, NO, YES, 768, 520, 392)):
    a, b, c = rnd(m * k), rnd(k * n), rnd(m * n)
    lda = (k if ta == NO else m) if layout == ROW else (m if ta == NO else k)
    ldb = (n if tb == NO else k) if layout == ROW else (k if tb == NO else n)
    ldc = n if layout == ROW else m
    assert cb.Gemm(layout, ta, tb, m, n, k, 0.7, a, 0, lda, b, 0, ldb, 0.3, c, 0, ldc) == 0
    out.append((cb.last_kernel(), c))
m, n, k, batch = 48, 200, 72, 400
a, b, c = rnd(batch * m * k), rnd(batch * k * n), rnd(batch * m * n)
assert cb.GemmStridedBatched(COL, NO, NO, m, n, k, 1.0, a, 0, m, m * k, b, 0, k, k * n, 1.0, c, 0, m, m * n, batch) == 0
out.append((cb.last_kernel(), c))
im, ker = rnd(8 * 32 * 40 * 37), rnd(96 * 32 * 9)
res = torch.zeros(8 * 96 * 40 * 37, device="cuda")
assert cb.Convgemm(151, 32, 40, 37, 3, 3, 1, 1, 1, 1, 1, 1, 96, 8, im, 0, ker, 0, res, 0) == 0
out.append((cb.last_kernel(), res))
torch.cuda.synchronize()
for name, t in out:
    print(name, hashlib.sha256(t.cpu().numpy().tobytes()).hexdigest())
"""


def test_tensor_memory_and_shared_memory_variants_agree_bit_for_bit(cuda):
    """The kernels that keep op(A) in tensor memory and the ones that keep it in shared memory (B200BLAS_SGEMM_TMEM_A=0)
    run the same MMAs in the same order on the same TF32 parts: identical bits on 128 x 64 and 128 x 128 tiles, a
    narrow batch and a convolution. Each variant runs in a process of its own (the switch is read once)."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    runs = {}
    for switch in ("1", "0"):
        # split-K adds the two halves of K in another order, so it is switched off for the comparison of bits
        env = dict(os.environ, B200BLAS_SGEMM_TMEM_A=switch, B200BLAS_SGEMM_SPLITK="0", PYTHONPATH=str(root))
        res = subprocess.run([sys.executable, "-c", _VARIANT_SCRIPT], capture_output=True, text=True, env=env, cwd=root,
                             timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        runs[switch] = [line.split() for line in res.stdout.strip().splitlines()]
    assert len(runs["1"]) == len(runs["0"]) == 5
    for (name_tm, digest_tm), (name_sm, digest_sm) in zip(runs["1"], runs["0"]):
        assert name_tm.endswith("_tmem_a") and name_tm.startswith(("tc_f32", "tc_conv")), name_tm
        assert not name_sm.endswith("_tmem_a") and name_sm.startswith(("tc_f32", "tc_conv")), name_sm
        assert digest_tm == digest_sm, (name_tm, name_sm)


@pytest.mark.parametrize("layout,ta,tb", ALL)
def test_few_tiles_split_k_over_a_cluster(cuda, layout, ta, tb):
    """Problems with so few 128 x 128 tiles that half the SMs would idle run as clusters of two CTAs that take half of
    K each and add their sums through distributed shared memory: every orientation, ragged extents, an odd number of
    K blocks, offsets and padded leading dimensions, beta = 0 on NaN-poisoned C."""
    rng = np.random.default_rng(31)
    run_tc32(cuda, rng, layout, ta, tb, 1024, 1024, 1024, 0.7, 0.3)
    assert cb.last_kernel() == "tc_f32_3xtf32_128x128x32_splitk2_tmem_a", cb.last_kernel()
    run_tc32(cuda, rng, layout, ta, tb, 700, 520, 1064, -1.25, 0.0, offs=(8, 4, 12), pad=(4, 8, 4))  # 34 K blocks, 33.25 used
    assert cb.last_kernel() == "tc_f32_3xtf32_128x128x32_splitk2_tmem_a", cb.last_kernel()
    run_tc32(cuda, rng, layout, ta, tb, 516, 300, 2000 + 36, 1.0, 1.0)  # 63.6 K blocks: an odd count, ragged tail
    assert cb.last_kernel() == "tc_f32_3xtf32_128x128x32_splitk2_tmem_a", cb.last_kernel()
