"""Parity of GemmStridedBatched and GemmBatched against a loop of single oracle GEMMs, which is how the reference's
own tests define them (test/routines/levelx/xgemmstridedbatched.hpp:131-141, xgemmbatched.hpp:154-162)."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu
ALL_PRECISIONS = (32, 64, 16, 3232, 6464)


def strided_case(rng, precision, layout, ta, tb, m, n, k, batch, pad=0, off=0, lo=-2.0, hi=2.0):
    a_one, a_two = H.stored_extents(layout, ta, m, k)
    b_one, b_two = H.stored_extents(layout, tb, k, n)
    c_one, c_two = H.stored_extents(layout, H.NO, m, n)
    g = dict(a_ld=a_one + pad, b_ld=b_one + pad, c_ld=c_one + pad)
    g["a_stride"] = g["a_ld"] * a_two + pad
    g["b_stride"] = g["b_ld"] * b_two + pad
    g["c_stride"] = g["c_ld"] * c_two + pad
    for key in "abc":
        g[key] = H.rand_buffer(rng, precision, off + g[key + "_stride"] * batch + H.CANARY, lo, hi)
    return g


def check_strided(torch, rng, precision, layout, ta, tb, m, n, k, batch, alpha, beta, pad=0, off=0, lo=-2.0, hi=2.0):
    g = strided_case(rng, precision, layout, ta, tb, m, n, k, batch, pad, off, lo, hi)
    da, db, dc = (H.to_device(torch, precision, g[x]) for x in "abc")
    torch.cuda.synchronize()
    st = cb.GemmStridedBatched(layout, ta, tb, m, n, k, alpha, da, off, g["a_ld"], g["a_stride"], db, off, g["b_ld"],
                               g["b_stride"], beta, dc, off, g["c_ld"], g["c_stride"], batch, precision=precision)
    assert st == cb.StatusCode.kSuccess, st
    got = H.to_host(precision, dc)
    want = oracle.widen(precision, g["c"])
    mask = np.zeros(g["c"].size, dtype=bool)
    for i in range(batch):
        want = _step(precision, layout, ta, tb, m, n, k, alpha, beta, g, off, i, want)
        mask |= H.c_mask(layout, m, n, off + i * g["c_stride"], g["c_ld"], g["c"].size)
    H.check_against_oracle(precision, got, want, mask, g["c"])


def _step(precision, layout, ta, tb, m, n, k, alpha, beta, g, off, i, want64):
    """One batch of the fp64 oracle, accumulated into the widened result image."""
    out = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alpha, g["a"], off + i * g["a_stride"], g["a_ld"],
                          g["b"], off + i * g["b_stride"], g["b_ld"], beta, g["c"], off + i * g["c_stride"], g["c_ld"])
    mask = H.c_mask(layout, m, n, off + i * g["c_stride"], g["c_ld"], g["c"].size)
    want64 = want64.copy()
    want64[mask] = out[mask]
    return want64


@pytest.mark.parametrize("precision", ALL_PRECISIONS)
def test_strided_batched_reference_grid(cuda, precision):
    rng = np.random.default_rng(42)
    trs = (H.NO, H.YES, H.CONJ) if precision > 100 else (H.NO, H.YES)
    i = 0
    for layout, ta, tb in itertools.product((H.ROW, H.COL), trs, trs):
        for (m, n, k), batch in zip(((7, 64, 7), (64, 7, 64), (64, 64, 7), (7, 7, 64)), (1, 3, 3, 1)):
            alpha, beta = ((3.14, 3.14), (1.0, 0.0), (1.0, 1.0))[i % 3]
            check_strided(cuda, rng, precision, layout, ta, tb, m, n, k, batch, alpha, beta, pad=i % 2 * 3,
                          off=i % 2 * 10)
            i += 1


@pytest.mark.parametrize("layout", (H.COL, H.ROW))
def test_config4_small_batched_shapes(cuda, layout):
    # the two strided-batched shapes of the benchmark configuration at a batch count the oracle finishes quickly,
    # then the full batch counts through a batch-independence property
    rng = np.random.default_rng(4)
    check_strided(cuda, rng, 32, layout, H.NO, H.NO, 32, 32, 32, 257, 1.0, 1.0, lo=-1, hi=1)
    check_strided(cuda, rng, 32, layout, H.NO, H.NO, 64, 128, 96, 65, 1.0, 1.0, lo=-1, hi=1)


@pytest.mark.parametrize("layout", (H.COL, H.ROW))
@pytest.mark.parametrize("ta,tb", ((H.NO, H.NO), (H.NO, H.YES), (H.YES, H.NO), (H.YES, H.YES)))
def test_streaming_small_batched_kernel(cuda, layout, ta, tb):
    """Large aligned batches of small fp32 problems take the cp.async streaming kernel; results must be bit-identical
    to the reference-order oracle, like the generic kernel's. The 64 x 128 x 96 class moves on to the tensor cores."""
    rng = np.random.default_rng(31)
    for (m, n, k), batch, (alpha, beta), pad in (((32, 32, 32), 301, (1.0, 1.0), 0), ((16, 24, 20), 600, (1.5, 0.0), 4),
                                                 ((64, 128, 96), 299, (1.0, 1.0), 0), ((60, 100, 64), 310, (0.5, 2.0), 8)):
        g = strided_case(rng, 32, layout, ta, tb, m, n, k, batch, pad, 0, -1, 1)
        da, db, dc = (H.to_device(cuda, 32, g[x]) for x in "abc")
        cuda.cuda.synchronize()
        st = cb.GemmStridedBatched(layout, ta, tb, m, n, k, alpha, da, 0, g["a_ld"], g["a_stride"], db, 0, g["b_ld"],
                                   g["b_stride"], beta, dc, 0, g["c_ld"], g["c_stride"], batch)
        assert st == cb.StatusCode.kSuccess
        mm, nn = (m, n) if layout == H.COL else (n, m)   # extents after normalisation to a column-major C
        got = H.to_host(32, dc)
        if mm <= 64 and nn >= 64 and k >= 32 and mm * nn * k * batch >= 2 ** 27:
            # narrow problems with enough columns go to the tensor cores as the transposed problem (3xTF32: fp32-level
            # accuracy, not the reference's order of operations)
            assert cb.last_kernel().startswith("tc_f32_3xtf32_narrow"), (cb.last_kernel(), m, n, k)
            want = oracle.widen(32, g["c"])
            for i in range(batch):
                out = oracle.gemm_f64(32, layout, ta, tb, m, n, k, alpha, g["a"], i * g["a_stride"], g["a_ld"], g["b"],
                                      i * g["b_stride"], g["b_ld"], beta, g["c"], i * g["c_stride"], g["c_ld"])
                one = H.c_mask(layout, m, n, i * g["c_stride"], g["c_ld"], g["c"].size)
                want[one] = out[one]
            assert np.abs(got - want).max() <= 2.0 ** -20 * (abs(alpha) * k + abs(beta))
            continue
        eligible = mm % 4 == 0 and ((mm <= 32 and nn <= 32 and k <= 32) or (mm <= 64 and nn <= 128 and k <= 96))
        assert cb.last_kernel().startswith("small_batched") == eligible, (cb.last_kernel(), m, n, k)
        want = g["c"].copy()
        for i in range(batch):
            oracle.gemm(32, layout, ta, tb, m, n, k, alpha, g["a"], i * g["a_stride"], g["a_ld"], g["b"],
                        i * g["b_stride"], g["b_ld"], beta, want, i * g["c_stride"], g["c_ld"])
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (m, n, k, layout, ta, tb)


def test_streaming_kernel_with_per_batch_tables(cuda):
    rng = np.random.default_rng(32)
    m = n = k = 32
    batch = 400
    per = m * k
    order = rng.permutation(batch)
    a_offs = [int(o * per) for o in order]
    b_offs = [int(o * per) for o in order[::-1]]
    c_offs = [int(o * per) for o in rng.permutation(batch)]
    a, b, c = (H.rand_buffer(rng, 32, batch * per, -1, 1) for _ in range(3))
    alphas = [1.0 + 0.01 * i for i in range(batch)]
    betas = [0.0 if i % 2 else 0.5 for i in range(batch)]
    da, db, dc = (H.to_device(cuda, 32, x) for x in (a, b, c))
    cuda.cuda.synchronize()
    assert cb.GemmBatched(H.COL, H.NO, H.NO, m, n, k, alphas, da, a_offs, m, db, b_offs, k, betas, dc, c_offs, m,
                          batch) == 0
    assert cb.last_kernel().startswith("small_batched")
    want = c.copy()
    for i in range(batch):
        oracle.gemm(32, H.COL, H.NO, H.NO, m, n, k, alphas[i], a, a_offs[i], m, b, b_offs[i], k, betas[i], want,
                    c_offs[i], m)
    assert np.array_equal(H.to_host(32, dc).view(np.uint8), want.view(np.uint8))
    # one offset that is not a multiple of 4 elements sends the whole call to the generic kernel
    a_offs[7] += 1
    a2 = np.concatenate([a, np.zeros(4, dtype=np.float32)])
    da2 = H.to_device(cuda, 32, a2)
    cuda.cuda.synchronize()
    assert cb.GemmBatched(H.COL, H.NO, H.NO, m, n, k, alphas, da2, a_offs, m, db, b_offs, k, betas, dc, c_offs, m,
                          batch) == 0
    assert cb.last_kernel().startswith("simt_")


@pytest.mark.parametrize("m,n,k,batch", ((32, 32, 32, 8192), (64, 128, 96, 2048)))
def test_config4_full_batch_equals_per_batch_calls(cuda, m, n, k, batch):
    torch = cuda
    g = torch.Generator(device="cuda").manual_seed(batch)
    a = torch.rand(batch * m * k, generator=g, device="cuda") * 2 - 1
    b = torch.rand(batch * k * n, generator=g, device="cuda") * 2 - 1
    c0 = torch.rand(batch * m * n, generator=g, device="cuda") * 2 - 1
    c = c0.clone()
    torch.cuda.synchronize()
    st = cb.GemmStridedBatched(H.COL, H.NO, H.NO, m, n, k, 1.0, a, 0, m, m * k, b, 0, k, k * n, 1.0, c, 0, m, m * n,
                               batch)
    assert st == cb.StatusCode.kSuccess
    # every 97th batch recomputed alone must match bit for bit (same kernel, same order of operations)
    for i in range(0, batch, 97):
        ci = c0[i * m * n:(i + 1) * m * n].clone()
        torch.cuda.synchronize()
        assert cb.Gemm(H.COL, H.NO, H.NO, m, n, k, 1.0, a, i * m * k, m, b, i * k * n, k, 1.0, ci, 0, m) == 0
        want = (b[i * k * n:(i + 1) * k * n].view(n, k).double() @ a[i * m * k:(i + 1) * m * k].view(k, m).double()
                + c0[i * m * n:(i + 1) * m * n].view(n, m).double())
        got = c[i * m * n:(i + 1) * m * n].view(n, m).double()
        assert torch.allclose(got, want, atol=1e-4, rtol=1e-5)
        assert torch.allclose(ci.view(n, m).double(), want, atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("precision", ALL_PRECISIONS)
def test_gemm_batched_with_per_batch_scalars_and_offsets(cuda, precision):
    torch = cuda
    rng = np.random.default_rng(precision)
    trs = (H.NO, H.YES, H.CONJ) if precision > 100 else (H.NO, H.YES)
    for layout, ta, tb, (m, n, k), batch in zip(itertools.cycle((H.COL, H.ROW)), itertools.cycle(trs),
                                                itertools.cycle(trs[::-1]),
                                                ((7, 64, 7), (64, 7, 64), (64, 64, 64), (33, 70, 129), (200, 130, 40)),
                                                (1, 3, 5, 4, 3)):
        a_one, a_two = H.stored_extents(layout, ta, m, k)
        b_one, b_two = H.stored_extents(layout, tb, k, n)
        c_one, c_two = H.stored_extents(layout, H.NO, m, n)
        a_ld, b_ld, c_ld = a_one + 1, b_one + 2, c_one + 3
        # batches are stored in a shuffled order with gaps, so offsets are neither sorted nor regular
        order = rng.permutation(batch)
        a_offs = [int(7 + o * (a_ld * a_two + 5)) for o in order]
        b_offs = [int(3 + o * (b_ld * b_two + 9)) for o in order[::-1]]
        c_offs = [int(11 + o * (c_ld * c_two + 2)) for o in rng.permutation(batch)]
        a = H.rand_buffer(rng, precision, max(a_offs) + a_ld * a_two + H.CANARY)
        b = H.rand_buffer(rng, precision, max(b_offs) + b_ld * b_two + H.CANARY)
        c = H.rand_buffer(rng, precision, max(c_offs) + c_ld * c_two + H.CANARY)
        alphas = [1.0 + 0.5 * i for i in range(batch)]
        betas = [0.0 if i % 2 else 0.75 for i in range(batch)]
        if precision > 100:
            alphas = [x + 0.25j for x in alphas]
        da, db, dc = (H.to_device(torch, precision, x) for x in (a, b, c))
        torch.cuda.synchronize()
        st = cb.GemmBatched(layout, ta, tb, m, n, k, alphas, da, a_offs, a_ld, db, b_offs, b_ld, betas, dc, c_offs,
                            c_ld, batch, precision=precision)
        assert st == cb.StatusCode.kSuccess, st
        got = H.to_host(precision, dc)
        want = oracle.widen(precision, c)
        mask = np.zeros(c.size, dtype=bool)
        for i in range(batch):
            out = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alphas[i], a, a_offs[i], a_ld, b, b_offs[i],
                                  b_ld, betas[i], c, c_offs[i], c_ld)
            mi = H.c_mask(layout, m, n, c_offs[i], c_ld, c.size)
            want[mi] = out[mi]
            mask |= mi
        H.check_against_oracle(precision, got, want, mask, c)
