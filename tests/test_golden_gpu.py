"""The CUDA path on the committed golden fixtures (inputs and float64 results made by tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def test_gemm_golden(cuda):
    data = np.load(GOLDEN / "gemm_cases.npz")
    for key in sorted({k.split("_")[0] for k in data.files}):
        precision, layout, ta, tb, m, n, k, a_off, a_ld, b_off, b_ld, c_off, c_ld = (int(x) for x in data[key + "_meta"])
        alpha, beta = data[key + "_scalars"]
        if precision < 100:
            alpha, beta = alpha.real, beta.real
        a, b, c, want = (data[key + s] for s in ("_a", "_b", "_c", "_want"))
        da, db, dc = (H.to_device(cuda, precision, np.ascontiguousarray(x)) for x in (a, b, c))
        cuda.cuda.synchronize()
        st = cb.Gemm(layout, ta, tb, m, n, k, alpha, da, a_off, a_ld, db, b_off, b_ld, beta, dc, c_off, c_ld,
                     precision=precision)
        assert st == cb.StatusCode.kSuccess, (key, st)
        got = H.to_host(precision, dc)
        r, cc = np.arange(m)[:, None], np.arange(n)[None, :]
        idx = c_off + (r * c_ld + cc if layout == 101 else cc * c_ld + r)
        bad, worst = oracle.count_mismatches(precision, got[idx], want.astype(oracle.widen(precision, c).dtype))
        assert bad == 0, (key, worst)
        mask = np.zeros(c.size, dtype=bool)
        mask[idx.ravel()] = True
        assert np.array_equal(got[~mask].view(np.uint8), c[~mask].view(np.uint8)), key


def test_conv_golden(cuda):
    data = np.load(GOLDEN / "conv_cases.npz")
    for key in sorted({k.split("_")[0] for k in data.files}):
        mode, ch, h, w, kh, kw, pad, stride, dil, nk, batch, oh, ow = (int(x) for x in data[key + "_meta"])
        im, ker, want = data[key + "_im"], data[key + "_ker"], data[key + "_want"]
        res = cuda.full((batch * nk * oh * ow,), float("nan"), device="cuda")
        dim, dker = cuda.from_numpy(im).cuda(), cuda.from_numpy(ker).cuda()
        cuda.cuda.synchronize()
        assert cb.Convgemm(mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, dim, 0, dker, 0, res,
                           0) == cb.StatusCode.kSuccess
        bad, worst = oracle.count_mismatches(32, res.cpu().numpy(), want.ravel())
        assert bad == 0, (key, worst)
        assert np.abs(res.cpu().numpy() - want.ravel()).max() < 1e-4
