"""Host-side sharding logic, including a world_size-2 run over gloo on CPU in which the oracle stands in for the
per-GPU Gemm call."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

from clblast_b200 import multi_gpu as mg

ROOT = Path(__file__).resolve().parent.parent


def test_split_range_covers_everything_with_aligned_boundaries():
    for total, parts, align in ((8192, 8, 256), (65536, 4, 256), (1000, 3, 256), (5, 8, 1), (0, 2, 4), (4097, 2, 256)):
        blocks = mg.split_range(total, parts, align)
        assert len(blocks) == parts
        assert blocks[0][0] == 0 and blocks[-1][1] == total
        for (s0, e0), (s1, e1) in zip(blocks, blocks[1:]):
            assert e0 == s1 and s0 <= e0
        for s, e in blocks[:-1]:
            assert e % align == 0 or e == total
        sizes = [e - s for s, e in blocks]
        assert sum(sizes) == total and max(sizes) <= -(-total // (parts * align)) * align


def test_column_shard_offsets():
    sh = mg.column_shard(n=8192, b_offset=5, b_ld=8200, c_offset=7, c_ld=8300, world=4, rank=2, align=256)
    assert (sh.j0, sh.n) == (4096, 2048)
    assert sh.b_offset == 5 + 4096 * 8200 and sh.c_offset == 7 + 4096 * 8300
    assert mg.batch_shard(10, 4, 0) == (0, 3) and mg.batch_shard(10, 4, 3) == (8, 2)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist
    from oracle import cpu_oracle as oracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, n, k = 40, 70, 30
    rng = np.random.default_rng(5)  # same seed everywhere: B and C are "resident" on every rank
    a_full = rng.uniform(-1, 1, m * k).astype(np.float32)
    b = rng.uniform(-1, 1, k * n).astype(np.float32)
    c = rng.uniform(-1, 1, m * n).astype(np.float32)
    a = torch.from_numpy(a_full.copy() if rank == 0 else np.zeros_like(a_full))  # only the owner holds A

    def gemm(layout, ta, tb, m_, n_, k_, alpha, a_buf, a_off, a_ld, b_buf, b_off, b_ld, beta, c_buf, c_off, c_ld):
        oracle.gemm(32, layout, ta, tb, m_, n_, k_, alpha, a_buf.numpy(), a_off, a_ld, b_buf, b_off, b_ld, beta, c_buf,
                    c_off, c_ld)
        return 0

    st, shard = mg.gemm_column_sharded(gemm, lambda buf, owner: dist.broadcast(buf, src=owner), world, rank, 0, 102,
                                       111, m, n, k, 1.5, a, 0, m, b, 0, k, 0.5, c, 0, m, align=16)
    assert st == 0
    np.save(os.path.join(out_dir, f"c_{rank}.npy"), c)
    np.save(os.path.join(out_dir, f"shard_{rank}.npy"), np.array([shard.j0, shard.n]))
    # batched split needs no communication
    b0, nb = mg.batch_shard(7, world, rank)
    np.save(os.path.join(out_dir, f"batch_{rank}.npy"), np.array([b0, nb]))
    dist.barrier()
    dist.destroy_process_group()


def test_column_sharded_gemm_over_gloo(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    world = 2
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    from oracle import cpu_oracle as oracle
    m, n, k = 40, 70, 30
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, m * k).astype(np.float32)
    b = rng.uniform(-1, 1, k * n).astype(np.float32)
    c0 = rng.uniform(-1, 1, m * n).astype(np.float32)
    want = c0.copy()
    oracle.gemm(32, 102, 111, 111, m, n, k, 1.5, a, 0, m, b, 0, k, 0.5, want, 0, m)
    covered = 0
    for r in range(world):
        j0, nn = np.load(tmp_path / f"shard_{r}.npy")
        c = np.load(tmp_path / f"c_{r}.npy")
        # the rank's own columns hold the result, all other columns are untouched
        assert np.array_equal(c[j0 * m:(j0 + nn) * m], want[j0 * m:(j0 + nn) * m])
        untouched = np.ones(m * n, dtype=bool)
        untouched[j0 * m:(j0 + nn) * m] = False
        assert np.array_equal(c[untouched], c0[untouched])
        covered += nn
    assert covered == n
    batches = [tuple(np.load(tmp_path / f"batch_{r}.npy")) for r in range(world)]
    assert batches == [(0, 4), (4, 3)]


def test_binomial_tree_reaches_every_rank_once():
    from clblast_b200.multi_gpu import binomial_tree
    for world in (1, 2, 3, 4, 5, 8, 13):
        for root in (0, world - 1):
            parents = {}
            for r in range(world):
                parent, children = binomial_tree(world, r, root)
                parents[r] = parent
                for c in children:
                    assert binomial_tree(world, c, root)[0] == r     # both sides agree on every edge
            assert parents[root] is None
            assert sum(p is None for p in parents.values()) == 1
            depth = 0
            for r in range(world):                                   # every rank reaches the root
                hops, x = 0, r
                while parents[x] is not None:
                    x = parents[x]
                    hops += 1
                    assert hops <= world
                assert x == root
                depth = max(depth, hops)
            assert depth <= (world - 1).bit_length()
    assert binomial_tree(8, 0) == (None, [4, 2, 1])
    assert binomial_tree(8, 4) == (0, [6, 5])
