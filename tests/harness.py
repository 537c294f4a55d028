"""Shared helpers of the parity tests: seeded host data, device round trips, comparison against the oracle."""
from __future__ import annotations

import numpy as np

from oracle import cpu_oracle as oracle

ROW, COL = 101, 102
NO, YES, CONJ = 111, 112, 113
CANARY = 127  # extra elements after every buffer, as in the reference's harness (src/utilities/utilities.hpp:46)

NP_OF = oracle.NP_OF
TORCH_NAME = {16: "float16", 32: "float32", 64: "float64", 3232: "complex64", 6464: "complex128"}


def rand_buffer(rng, precision, size, lo=-2.0, hi=2.0):
    """Uniform data in [lo, hi) in the routine's type (the reference draws from U[-2, 2], testblas.cpp:84-92)."""
    x = rng.uniform(lo, hi, size)
    if precision in (3232, 6464):
        x = x + 1j * rng.uniform(lo, hi, size)
    return x.astype(NP_OF[precision])


def stored_extents(layout, trans, rows, cols):
    """(contiguous extent, other extent) of a stored matrix whose op() is rows x cols."""
    r, c = (rows, cols) if trans == NO else (cols, rows)
    return (c, r) if layout == ROW else (r, c)


def buffer_size(one, two, ld, offset):
    return ld * (two - 1) + one + offset


def to_device(torch, precision, host: np.ndarray):
    t = torch.from_numpy(host.view(np.float16) if precision == 16 else host)
    return t.cuda()


def to_host(precision, dev) -> np.ndarray:
    return dev.cpu().numpy()


def gemm_case(rng, precision, layout, ta, tb, m, n, k, a_off=0, b_off=0, c_off=0, ld_pad=(0, 0, 0), lo=-2.0, hi=2.0,
              poison_c=False):
    """Host buffers (with canary tails) and geometry for one GEMM call."""
    a_one, a_two = stored_extents(layout, ta, m, k)
    b_one, b_two = stored_extents(layout, tb, k, n)
    c_one, c_two = stored_extents(layout, NO, m, n)
    a_ld, b_ld, c_ld = a_one + ld_pad[0], b_one + ld_pad[1], c_one + ld_pad[2]
    a = rand_buffer(rng, precision, buffer_size(a_one, a_two, a_ld, a_off) + CANARY, lo, hi)
    b = rand_buffer(rng, precision, buffer_size(b_one, b_two, b_ld, b_off) + CANARY, lo, hi)
    c = rand_buffer(rng, precision, buffer_size(c_one, c_two, c_ld, c_off) + CANARY, lo, hi)
    if poison_c:
        c[:] = np.nan
    return dict(a=a, b=b, c=c, a_ld=a_ld, b_ld=b_ld, c_ld=c_ld, a_off=a_off, b_off=b_off, c_off=c_off)


def c_mask(layout, m, n, c_off, c_ld, size):
    """Boolean mask of the C-buffer elements the routine is allowed to write."""
    mask = np.zeros(size, dtype=bool)
    one, two = (n, m) if layout == ROW else (m, n)
    idx = (c_off + np.arange(two)[:, None] * c_ld + np.arange(one)[None, :]).ravel()
    mask[idx] = True
    return mask


def check_against_oracle(precision, got: np.ndarray, want64: np.ndarray, mask: np.ndarray, before: np.ndarray,
                         scale64: np.ndarray | None = None):
    """Asserts (1) the reference's similarity rule on every written element versus the fp64 oracle, (2) no element
    outside the routine's footprint changed (padding and canary), and returns the worst absolute error."""
    bad, worst = oracle.count_mismatches(precision, got[mask], want64[mask])
    assert bad == 0, f"{bad} elements outside the reference's margins (worst abs diff {worst:.3e})"
    outside = ~mask
    same = (got[outside].view(np.uint8) == before[outside].view(np.uint8))
    assert same.all(), "elements outside the C footprint were modified"
    return worst
