"""The allocation-free GemmBatched entry point against the regular one.

Some callers cannot allocate device memory at call time (their own arena owns the whole GPU, or they sit in a
latency-critical loop), so b200blas_gemm_batched_static keeps its per-batch tables in a fixed array inside the
library. This test calls it twice in a row through the C ABI with different shapes, scalars and offsets (the second
call must not see anything of the first call's tables) and requires bit-identical results to
b200blas_gemm_batched, which runs the same kernels. It is collected last on purpose, and passes alone as well."""
import numpy as np
import pytest

import clblast_b200 as cb
from clblast_b200.api import STATIC_MAX_BATCHES
from tests import harness as H

pytestmark = pytest.mark.gpu


def _case(rng, precision, m, n, k, batch):
    a_ld, b_ld, c_ld = m + 1, k + 2, m + 3
    order = rng.permutation(batch)
    a_offs = [int(5 + o * (a_ld * k + 3)) for o in order]
    b_offs = [int(2 + o * (b_ld * n + 7)) for o in order[::-1]]
    c_offs = [int(9 + o * (c_ld * n + 1)) for o in rng.permutation(batch)]
    a = H.rand_buffer(rng, precision, max(a_offs) + a_ld * k + H.CANARY)
    b = H.rand_buffer(rng, precision, max(b_offs) + b_ld * n + H.CANARY)
    c = H.rand_buffer(rng, precision, max(c_offs) + c_ld * n + H.CANARY)
    alphas = [0.5 + 0.25 * i for i in range(batch)]
    betas = [0.0 if i % 3 == 0 else 1.0 + 0.125 * i for i in range(batch)]
    if precision > 100:
        alphas = [x - 0.5j for x in alphas]
    return dict(a=a, b=b, c=c, a_ld=a_ld, b_ld=b_ld, c_ld=c_ld, a_offs=a_offs, b_offs=b_offs, c_offs=c_offs,
                alphas=alphas, betas=betas)


def test_static_table_variant_matches_the_allocating_one_on_two_calls_in_a_row(cuda):
    torch = cuda
    rng = np.random.default_rng(2024)
    stream = torch.cuda.Stream()
    # second call: another precision (wider scalars), a smaller batch count and other offsets
    for precision, (m, n, k), batch in ((32, (33, 70, 129), 37), (6464, (20, 17, 40), 5), (16, (64, 64, 64), 200)):
        g = _case(rng, precision, m, n, k, batch)
        da, db = H.to_device(torch, precision, g["a"]), H.to_device(torch, precision, g["b"])
        dc_ref, dc_new = H.to_device(torch, precision, g["c"]), H.to_device(torch, precision, g["c"])
        torch.cuda.synchronize()
        args = (H.COL, H.NO, H.NO, m, n, k, g["alphas"], da, g["a_offs"], g["a_ld"], db, g["b_offs"], g["b_ld"],
                g["betas"])
        assert cb.GemmBatched(*args, dc_ref, g["c_offs"], g["c_ld"], batch, precision=precision) == 0
        assert cb.GemmBatchedStatic(*args, dc_new, g["c_offs"], g["c_ld"], batch, precision=precision, stream=stream,
                                    wait=True) == 0
        ref, new = H.to_host(precision, dc_ref), H.to_host(precision, dc_new)
        assert np.array_equal(ref.view(np.uint8), new.view(np.uint8)), precision
        assert not np.array_equal(ref.view(np.uint8), g["c"].view(np.uint8))  # something was computed


def test_static_table_variant_rejects_oversized_batches(cuda):
    torch = cuda
    batch = STATIC_MAX_BATCHES + 1
    buf = torch.zeros(64, device="cuda")
    st = cb.GemmBatchedStatic(H.COL, H.NO, H.NO, 2, 2, 2, [1.0] * batch, buf, [0] * batch, 2, buf, [0] * batch, 2,
                              [0.0] * batch, buf, [0] * batch, 2, batch, stream=torch.cuda.current_stream())
    assert st == cb.StatusCode.kInvalidBatchCount


def test_static_table_variant_on_evenly_spaced_offsets_reaches_the_tensor_cores(cuda):
    """Evenly spaced offset tables are recognised on the host and run on the tensor-core kernels; the result is
    compared with the regular entry point (bit for bit) and directly with the fp64 oracle, two calls in a row."""
    from oracle import cpu_oracle as oracle
    torch = cuda
    rng = np.random.default_rng(77)
    stream = torch.cuda.Stream()
    for m, n, k, batch in ((256, 256, 256, 12), (512, 256, 192, 6)):
        a_offs = [i * m * k for i in range(batch)]
        b_offs = [i * k * n for i in range(batch)]
        c_offs = [i * m * n for i in range(batch)]
        a = H.rand_buffer(rng, 32, batch * m * k, -1, 1)
        b = H.rand_buffer(rng, 32, batch * k * n, -1, 1)
        c = H.rand_buffer(rng, 32, batch * m * n, -1, 1)
        alphas = [1.0 + 0.25 * i for i in range(batch)]
        betas = [0.5 if i % 2 else 0.0 for i in range(batch)]
        da, db = H.to_device(torch, 32, a), H.to_device(torch, 32, b)
        dc_ref, dc_new = H.to_device(torch, 32, c), H.to_device(torch, 32, c)
        torch.cuda.synchronize()
        args = (H.COL, H.NO, H.NO, m, n, k, alphas, da, a_offs, m, db, b_offs, k, betas)
        assert cb.GemmBatched(*args, dc_ref, c_offs, m, batch, precision=32) == 0
        assert cb.GemmBatchedStatic(*args, dc_new, c_offs, m, batch, precision=32, stream=stream, wait=True) == 0
        assert cb.last_kernel().startswith("tc_"), cb.last_kernel()
        ref, new = H.to_host(32, dc_ref), H.to_host(32, dc_new)
        assert np.array_equal(ref.view(np.uint8), new.view(np.uint8))
        for i in (0, batch - 1):
            want = oracle.gemm_f64(32, H.COL, H.NO, H.NO, m, n, k, alphas[i], a, a_offs[i], m, b, b_offs[i], k, betas[i],
                                   c, c_offs[i], m)
            sl = slice(c_offs[i], c_offs[i] + m * n)
            bad, worst = oracle.count_mismatches(32, new[sl], want[sl])
            assert bad == 0, (i, worst)
            assert worst / (alphas[i] * k + 1.0) < 2.0 ** -20


def test_static_table_variant_refuses_a_capturing_stream(cuda):
    torch = cuda
    buf = torch.zeros(64, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    before = cb.launch_count()
    with torch.cuda.graph(graph, stream=side):
        st = cb.GemmBatchedStatic(H.COL, H.NO, H.NO, 2, 2, 2, [1.0], buf, [0], 2, buf, [8], 2, [0.0], buf, [16], 2, 1,
                                  stream=side, wait=False)
    assert st == cb.StatusCode.kUnexpectedError
    assert cb.launch_count() == before  # nothing was enqueued
    torch.cuda.synchronize()
    assert float(buf.abs().sum()) == 0.0
