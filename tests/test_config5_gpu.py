"""The sharded configuration: DGEMM 32768^3 and SGEMM 65536^3, column-major, not transposed, alpha 1, beta 0.

The reference cannot address these matrices at all: it casts sizes and offsets to 32-bit int
(src/routines/level3/xgemm.cpp:195-204) and 65536^2 elements is 2^32. Here the whole product runs on one GPU, and
once more with the arguments rank 7 of 8 passes when C is split by column blocks (n = N/8, B and C addressed through
offset += j0 * ld, which puts the offsets themselves beyond 2^31 and, for SGEMM, next to 2^32).

Checked: C was poisoned with NaN and beta is 0, so no NaN may remain; a grid of sampled entries (rows and columns
forced into the first and last rows, the last column block and the last column, i.e. byte offsets above 2^32 and,
for SGEMM, element indices above 2^32 - ld) is compared with exact fp64 dot products of length K under the reference's own margins
(test/correctness/tester.cpp:29-69) and the tight normalised bounds used for the small cases."""
import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu

TIGHT = {32: 2.0 ** -20, 64: 2.0 ** -48}


def _fill(torch, count, dt, gen):
    """U[-1, 1) of `count` elements, generated in slices (torch.rand materialises temporaries)."""
    out = torch.empty(count, device="cuda", dtype=dt)
    step = 1 << 28
    for s0 in range(0, count, step):
        e0 = min(count, s0 + step)
        out[s0:e0] = torch.rand(e0 - s0, generator=gen, device="cuda", dtype=dt) * 2 - 1
    return out


def _sample_grid(rng, n, forced_rows, forced_cols, count=64):
    """Sorted row and column indices: the forced ones plus random ones up to `count` each."""
    def pick(forced):
        forced = np.unique(np.asarray(forced))
        extra = np.setdiff1d(rng.permutation(n)[:4 * count], forced)[:count - len(forced)]
        return np.sort(np.concatenate([forced, extra])).astype(np.int64)
    return pick(forced_rows), pick(forced_cols)


def _check(torch, precision, a, b, c, n, rows, cols):
    """Compares C(rows x cols) with fp64 dot products. Only the sampled rows of A and columns of B leave the GPU."""
    r_t = torch.from_numpy(rows).cuda()
    c_t = torch.from_numpy(cols).cuda()
    k_idx = torch.arange(n, device="cuda", dtype=torch.int64)
    # A is n x n column-major: row i is the strided set {i + l*n}; B's column j is contiguous
    a_rows = a[(r_t[:, None] + k_idx[None, :] * n).reshape(-1)].cpu().numpy().reshape(len(rows), n)
    b_cols = b[(c_t[:, None] * n + k_idx[None, :]).reshape(-1)].cpu().numpy().reshape(len(cols), n)
    got = c[(c_t[None, :] * n + r_t[:, None]).reshape(-1)].cpu().numpy().astype(np.float64)
    # the compact operands as a small column-major problem: A_s is len(rows) x n (row-contiguous here, so it is passed
    # as a transposed operand), B_s is n x len(cols)
    rr, cc = np.meshgrid(np.arange(len(rows)), np.arange(len(cols)), indexing="ij")
    want, mag = oracle.gemm_f64_sampled(precision, H.COL, H.YES, H.NO, n, 1.0, np.ascontiguousarray(a_rows).ravel(), 0, n,
                                        np.ascontiguousarray(b_cols).ravel(), 0, n, rr.ravel(), cc.ravel())
    assert np.isfinite(got).all()
    bad, worst = oracle.count_mismatches(precision, got, want)
    assert bad == 0, worst
    err = (np.abs(got - want) / mag).max()
    assert err < TIGHT[precision], err
    return err


@pytest.mark.parametrize("precision,n", ((64, 32768), (32, 65536)))
def test_config5_full_product_and_last_rank_shard(cuda, precision, n):
    torch = cuda
    dt = getattr(torch, H.TORCH_NAME[precision])
    elem = 8 if precision == 64 else 4
    need = 3 * n * n * elem + (6 << 30)
    free, _total = torch.cuda.mem_get_info()
    assert free > need, f"needs {need >> 30} GiB of device memory, {free >> 30} GiB free"
    gen = torch.Generator(device="cuda").manual_seed(n)
    a = _fill(torch, n * n, dt, gen)
    b = _fill(torch, n * n, dt, gen)
    c = torch.full((n * n,), float("nan"), device="cuda", dtype=dt)
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, n, n, n, 1.0, a, 0, n, b, 0, n, 0.0, c, 0, n) == cb.StatusCode.kSuccess
    kernel = cb.last_kernel()
    assert kernel.startswith("tc_f32_3xtf32_pair") if precision == 32 else kernel.startswith("dmma_f64"), kernel
    step = 1 << 30
    for s0 in range(0, n * n, step):
        assert not bool(torch.isnan(c[s0:s0 + step]).any()), "C keeps poisoned entries"
    rng = np.random.default_rng(n)
    rows, cols = _sample_grid(rng, n, (0, 1, 127, 128, n - 129, n - 2, n - 1), (0, 255, 256, n - 257, n - 256, n - 2, n - 1))
    last = int(cols[-1]) * n + int(rows[-1])            # element index of the last sample
    assert last == n * n - 1 and last * elem >= (1 << 32)   # byte offsets beyond 32 bits in both cases
    if precision == 32:
        assert last >= (1 << 32) - n                        # and element indices that no 32-bit integer holds
    _check(torch, precision, a, b, c, n, rows, cols)

    # rank 7 of 8: its column block through the offset arguments, into a fresh C of the block's size
    from clblast_b200.multi_gpu import column_shard
    shard = column_shard(n, 0, n, 0, n, 8, 7)
    assert shard.n == n // 8 and shard.b_offset == shard.j0 * n and shard.b_offset * elem >= (1 << 32)
    c.fill_(float("nan"))
    torch.cuda.synchronize()
    assert cb.Gemm(H.COL, H.NO, H.NO, n, shard.n, n, 1.0, a, 0, n, b, shard.b_offset, n, 0.0, c, shard.c_offset,
                   n) == cb.StatusCode.kSuccess
    lo, hi = shard.c_offset, shard.c_offset + shard.n * n
    assert bool(torch.isnan(c[lo - (1 << 20):lo]).all()) and not bool(torch.isnan(c[lo:lo + (1 << 24)]).any())
    assert hi == n * n and not bool(torch.isnan(c[hi - (1 << 24):hi]).any())
    cols7 = cols[cols >= shard.j0]
    cols7 = np.unique(np.concatenate([cols7, np.asarray([shard.j0, shard.j0 + 1, n - 1])]))
    _check(torch, precision, a, b, c, n, rows, cols7)
