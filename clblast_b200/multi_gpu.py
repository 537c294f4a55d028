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


# ---- replication of the unsplit operand with the copy engines ---------------------------------------------------

def binomial_tree(world: int, rank: int, root: int = 0):
    """(parent, children) of ``rank`` in the binomial broadcast tree rooted at ``root``.

    Children are listed farthest first, the order in which a node forwards: with 8 ranks the root sends to 4, 2, 1;
    rank 4 to 6, 5; ranks 2 and 6 to 3 and 7. Every rank receives once; no rank is more than ceil(log2(world)) hops from the root."""
    if world < 1 or not 0 <= rank < world or not 0 <= root < world:
        raise ValueError("invalid world / rank / root")
    rel = (rank - root) % world
    parent = None
    mask = 1
    while mask < world:
        if rel & mask:
            parent = ((rel - mask) + root) % world
            break
        mask <<= 1
    children = []
    m = mask >> 1
    while m >= 1:
        if rel + m < world:
            children.append(((rel + m) + root) % world)
        m >>= 1
    return parent, children


class CopyEngineFanout:
    """Replicates a buffer from ``root`` to every rank of one node, step after step, without a collective kernel.

    Each rank owns a ring of ``len(buffers)`` equally sized device buffers. In step s (1, 2, ...) the contents of the
    root's ``buffers[s % depth]`` travel down a binomial tree: a node waits until its parent's copy has landed
    (a 32-bit flag in its own memory, waited for by the stream front-end), forwards the buffer to its children with
    ``cudaMemcpyAsync`` into their mapped memory (copy engines, NVLink), and raises their flags. A child tells its
    parent when it is done with a ring slot, so with two buffers the transfer of step s overlaps the compute of
    step s - 1 on every rank while the compute kernels keep all SMs and read local memory only.

    ``step_begin`` enqueues the step's forwarding on an internal copy stream and makes the compute stream wait for the
    step's data; ``step_end`` is called after the compute that reads the buffer has been enqueued."""

    MAX_STEPS = 1 << 16

    def __init__(self, dist, buffers, root: int = 0):
        import ctypes

        import torch

        from ._lib import lib

        self._ct, self._torch, self._L = ctypes, torch, lib()
        self.world, self.rank, self.root = dist.get_world_size(), dist.get_rank(), root
        self.depth = len(buffers)
        if self.depth < 1 or any(b.numel() * b.element_size() != buffers[0].numel() * buffers[0].element_size()
                                 for b in buffers):
            raise ValueError("the ring needs at least one buffer, all of one size")
        self.buffers = list(buffers)
        self.nbytes = buffers[0].numel() * buffers[0].element_size()
        self.parent, self.children = binomial_tree(self.world, self.rank, root)
        dev = buffers[0].device
        # word 0: newest step whose data has landed here; word 1 + i: newest step child i has finished with
        self.flags = torch.zeros(64, dtype=torch.int32, device=dev)
        self.seq = torch.arange(self.MAX_STEPS, dtype=torch.int32, device=dev)   # source words of the flag copies
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.step = 0
        self._fwd_done = None
        torch.cuda.synchronize(dev)

        mine = {"buffers": [self._export(b) for b in self.buffers], "flags": self._export(self.flags)}
        table = [None] * self.world
        dist.all_gather_object(table, mine)
        self._opened = {}
        self.child_buffers = [[self._open(table[c]["buffers"][i]) for i in range(self.depth)] for c in self.children]
        self.child_flags = [self._open(table[c]["flags"]) for c in self.children]
        self.parent_flags = self._open(table[self.parent]["flags"]) if self.parent is not None else None
        if self.parent is not None:
            _, siblings = binomial_tree(self.world, self.parent, root)
            self.slot_at_parent = 1 + siblings.index(self.rank)
        dist.barrier()

    def _export(self, tensor):
        handle = (self._ct.c_ubyte * 64)()
        offset = self._ct.c_size_t(0)
        st = self._L.b200blas_ipc_export(tensor.data_ptr(), handle, self._ct.byref(offset))
        if st != 0:
            raise RuntimeError(f"exporting a device allocation failed with status {st}")
        return bytes(handle), offset.value

    def _open(self, exported):
        handle, offset = exported
        if handle not in self._opened:   # one mapping per peer allocation, however many buffers live in it
            out = self._ct.c_void_p()
            raw = (self._ct.c_ubyte * 64).from_buffer_copy(handle)
            st = self._L.b200blas_ipc_open(raw, 0, self._ct.byref(out))
            if st != 0:
                raise RuntimeError(f"mapping a peer allocation failed with status {st}")
            self._opened[handle] = out.value
        return self._opened[handle] + offset

    def _check(self, st, what):
        if st != 0:
            raise RuntimeError(f"{what} failed with status {st}")

    def step_begin(self, compute_stream, ready_event=None):
        """Starts step ``self.step + 1``. On the root, ``ready_event`` (optional) marks the point where the step's
        buffer has been produced. Returns the local buffer that holds the step's data once ``compute_stream`` runs."""
        torch, L = self._torch, self._L
        self.step += 1
        s = self.step
        if s >= self.MAX_STEPS:
            raise RuntimeError("step counter exhausted")
        slot = s % self.depth
        cs = self.copy_stream.cuda_stream
        if self.parent is not None:
            self._check(L.b200blas_stream_wait_flag(cs, self.flags.data_ptr(), s), "stream wait")
            self._check(L.b200blas_stream_wait_flag(compute_stream.cuda_stream, self.flags.data_ptr(), s), "stream wait")
        elif ready_event is not None:
            self.copy_stream.wait_event(ready_event)
        for i, child in enumerate(self.children):
            if s > self.depth:   # the child must have finished with the slot's previous contents
                self._check(L.b200blas_stream_wait_flag(cs, self.flags.data_ptr() + 4 * (1 + i), s - self.depth),
                            "stream wait")
            self._check(L.b200blas_stream_copy(cs, self.child_buffers[i][slot], self.buffers[slot].data_ptr(),
                                               self.nbytes), "peer copy")
            self._check(L.b200blas_stream_copy(cs, self.child_flags[i], self.seq.data_ptr() + 4 * s, 4), "flag copy")
        if self.children:
            self._fwd_done = torch.cuda.Event()
            self._fwd_done.record(self.copy_stream)
        return self.buffers[slot]

    def step_end(self, compute_stream):
        """Releases the step's ring slot to the parent once the compute enqueued so far and this rank's own forwards
        of the step have finished."""
        if self.children and self._fwd_done is not None:
            compute_stream.wait_event(self._fwd_done)
        if self.parent is not None:
            self._check(self._L.b200blas_stream_copy(compute_stream.cuda_stream, self.parent_flags + 4 * self.slot_at_parent,
                                                     self.seq.data_ptr() + 4 * self.step, 4), "flag copy")

    def close(self):
        self._torch.cuda.synchronize()
        for base in self._opened.values():
            self._L.b200blas_ipc_close(base, 0)
        self._opened = {}
