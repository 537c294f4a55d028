"""Sharding of the GEMM family over the GPUs of one node, one process per GPU.

The reference is a single-device library (one context and one stream per call); this layer sits above the
unchanged per-device API and uses exactly what its offset / leading-dimension arguments allow:

* a large column-major GEMM is split by COLUMN BLOCKS of C: rank r computes
  ``C[:, j0:j1] = alpha * op(A) * op(B)[:, j0:j1] + beta * C[:, j0:j1]`` with ``n = j1 - j0`` and B and C
  addressed through ``offset += j0 * ld``. K is not split, so there is no reduction; the only exchange is that
  every rank needs all of A, which the owner broadcasts over NCCL into each rank's own memory;
* batched and strided-batched GEMMs and Convgemm are split by BATCH INDEX with no communication at all.

Kernels only ever read the local GPU's memory. The collective is injected (``broadcast``) so the same logic runs
under ``torch.distributed`` with NCCL on GPUs and with gloo on CPU in the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Tuple


def split_range(total: int, parts: int, align: int = 1) -> List[Tuple[int, int]]:
    """Splits [0, total) into ``parts`` contiguous blocks whose interior boundaries are multiples of ``align``.

    Blocks differ by at most one aligned unit; trailing blocks may be empty when total < parts * align."""
    if parts < 1 or align < 1 or total < 0:
        raise ValueError("parts and align must be positive and total non-negative")
    units = -(-total // align)
    base, extra = divmod(units, parts)
    bounds, start = [], 0
    for p in range(parts):
        end = min(total, start + (base + (1 if p < extra else 0)) * align)
        bounds.append((start, end))
        start = end
    return bounds


@dataclass
class ColumnShard:
    """What one rank passes to the single-GPU Gemm for its block of columns."""
    j0: int
    n: int
    b_offset: int
    c_offset: int


def column_shard(n: int, b_offset: int, b_ld: int, c_offset: int, c_ld: int, world: int, rank: int,
                 align: int = 256) -> ColumnShard:
    """Column block of rank ``rank`` for a column-major, B-not-transposed GEMM (B is K x N with columns b_ld apart)."""
    j0, j1 = split_range(n, world, align)[rank]
    return ColumnShard(j0=j0, n=j1 - j0, b_offset=b_offset + j0 * b_ld, c_offset=c_offset + j0 * c_ld)


def batch_shard(batch_count: int, world: int, rank: int) -> Tuple[int, int]:
    """(first batch, number of batches) of rank ``rank``."""
    b0, b1 = split_range(batch_count, world, 1)[rank]
    return b0, b1 - b0


def gemm_column_sharded(gemm: Callable, broadcast: Callable, world: int, rank: int, owner: int, layout, a_transpose,
                        m: int, n: int, k: int, alpha, a_buffer, a_offset: int, a_ld: int, b_buffer, b_offset: int,
                        b_ld: int, beta, c_buffer, c_offset: int, c_ld: int, align: int = 256, **gemm_kwargs):
    """Runs this rank's share of one column-major GEMM whose B is not transposed.

    ``a_buffer`` must be allocated on every rank and hold A on ``owner``; ``broadcast(buffer, owner)`` replicates it.
    ``b_buffer`` / ``c_buffer`` are this rank's full-geometry B and C (only the rank's column block is touched).
    ``gemm`` has the signature of :func:`clblast_b200.Gemm`. Returns (status, ColumnShard)."""
    if int(layout) != 102:
        raise ValueError("column sharding is defined for the column-major layout")
    if world > 1:
        broadcast(a_buffer, owner)
    shard = column_shard(n, b_offset, b_ld, c_offset, c_ld, world, rank, align)
    if shard.n == 0:
        return 0, shard
    status = gemm(layout, a_transpose, 111, m, shard.n, k, alpha, a_buffer, a_offset, a_ld, b_buffer, shard.b_offset,
                  b_ld, beta, c_buffer, shard.c_offset, c_ld, **gemm_kwargs)
    return status, shard


def gemm_strided_batched_sharded(gemm_strided_batched: Callable, world: int, rank: int, layout, a_transpose,
                                 b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld, a_stride, b_buffer, b_offset,
                                 b_ld, b_stride, beta, c_buffer, c_offset, c_ld, c_stride, batch_count,
                                 **kwargs):
    """Runs this rank's contiguous range of batches; no communication. Returns (status, first batch, count)."""
    b0, nb = batch_shard(batch_count, world, rank)
    if nb == 0:
        return 0, b0, 0
    status = gemm_strided_batched(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer,
                                  a_offset + b0 * a_stride, a_ld, a_stride, b_buffer, b_offset + b0 * b_stride, b_ld,
                                  b_stride, beta, c_buffer, c_offset + b0 * c_stride, c_ld, c_stride, nb, **kwargs)
    return status, b0, nb
