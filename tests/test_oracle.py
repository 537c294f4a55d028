"""The CPU oracle against the committed golden fixtures (numpy float64 results) and the reference's comparison rule."""
from pathlib import Path

import numpy as np
import pytest

from oracle import cpu_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def dense(buf, off, ld, m, n, layout):
    r, c = np.arange(m)[:, None], np.arange(n)[None, :]
    return buf[off + (r * ld + c if layout == 101 else c * ld + r)]


def test_gemm_oracle_matches_golden_fixtures():
    data = np.load(GOLDEN / "gemm_cases.npz")
    keys = sorted({k.split("_")[0] for k in data.files})
    assert len(keys) >= 40
    for key in keys:
        precision, layout, ta, tb, m, n, k, a_off, a_ld, b_off, b_ld, c_off, c_ld = (int(x) for x in data[key + "_meta"])
        alpha, beta = data[key + "_scalars"]
        if precision < 100:
            alpha, beta = alpha.real, beta.real
        a, b, c, want = (data[key + s] for s in ("_a", "_b", "_c", "_want"))
        # fp64 flavour: equal to numpy's product up to summation-order rounding
        c64 = oracle.gemm_f64(precision, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, c, c_off, c_ld)
        got = dense(c64, c_off, c_ld, m, n, layout)
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max()), key
        # untouched elements keep their widened input value
        touched = np.zeros(c.size, dtype=bool)
        r, cc = np.arange(m)[:, None], np.arange(n)[None, :]
        touched[(c_off + (r * c_ld + cc if layout == 101 else cc * c_ld + r)).ravel()] = True
        assert np.array_equal(c64[~touched], oracle.widen(precision, c)[~touched]), key
        # reference-order flavour in the routine's own type: within the reference's margins of the fp64 result
        ct = c.copy()
        oracle.gemm(precision, layout, ta, tb, m, n, k, alpha, a, a_off, a_ld, b, b_off, b_ld, beta, ct, c_off, c_ld)
        bad, _ = oracle.count_mismatches(precision, dense(ct, c_off, c_ld, m, n, layout), want.astype(c64.dtype))
        assert bad == 0, key
        assert np.array_equal(ct[~touched].view(np.uint8), c[~touched].view(np.uint8)), key


def test_conv_oracle_matches_golden_fixtures():
    data = np.load(GOLDEN / "conv_cases.npz")
    keys = sorted({k.split("_")[0] for k in data.files})
    assert len(keys) == 10
    for key in keys:
        mode, ch, h, w, kh, kw, pad, stride, dil, nk, batch, oh, ow = (int(x) for x in data[key + "_meta"])
        assert oracle.conv_output_size(h, w, kh, kw, pad, pad, stride, stride, dil, dil) == (oh, ow)
        im, ker, want = data[key + "_im"], data[key + "_ker"], data[key + "_want"]
        res = np.full(batch * nk * oh * ow, np.nan, dtype=np.float32)
        got64 = oracle.convgemm(32, mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, im, 0, ker, 0,
                                res, 0, f64=True)
        assert np.abs(got64 - want.ravel()).max() < 1e-12, key
        oracle.convgemm(32, mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, im, 0, ker, 0, res, 0)
        assert np.abs(res - want.ravel()).max() < 1e-5, key


def test_sampled_products_agree_with_the_full_oracle():
    rng = np.random.default_rng(0)
    m, n, k = 50, 40, 300
    for layout in (101, 102):
        for ta in (111, 112):
            for tb in (111, 112):
                a = rng.uniform(-1, 1, m * k).astype(np.float32)
                b = rng.uniform(-1, 1, k * n).astype(np.float32)
                a_ld = (k if ta == 111 else m) if layout == 101 else (m if ta == 111 else k)
                b_ld = (n if tb == 111 else k) if layout == 101 else (k if tb == 111 else n)
                c_ld = n if layout == 101 else m
                c = np.zeros(m * n, dtype=np.float32)
                full = oracle.gemm_f64(32, layout, ta, tb, m, n, k, 1.5, a, 0, a_ld, b, 0, b_ld, 0.0, c, 0, c_ld)
                rows, cols = rng.integers(0, m, 64), rng.integers(0, n, 64)
                vals, mag = oracle.gemm_f64_sampled(32, layout, ta, tb, k, 1.5, a, 0, a_ld, b, 0, b_ld, rows, cols)
                idx = rows * c_ld + cols if layout == 101 else cols * c_ld + rows
                assert np.allclose(vals, full[idx], rtol=1e-13, atol=1e-13)
                assert (mag >= np.abs(vals) / 1.5 - 1e-12).all()


def test_half_oracle_accumulates_in_half():
    # 2048 additions of 1.0 in half stop growing at 2048 (spacing 2 above it): the reference-order oracle shows it,
    # the fp64 yardstick does not
    k = 4096
    a = np.ones(k, dtype=np.float16)
    b = np.ones(k, dtype=np.float16)
    c = np.zeros(1, dtype=np.float16)
    oracle.gemm(16, 102, 111, 111, 1, 1, k, 1.0, a, 0, 1, b, 0, k, 0.0, c, 0, 1)
    assert float(c[0]) == 2048.0
    c64 = oracle.gemm_f64(16, 102, 111, 111, 1, 1, k, 1.0, a, 0, 1, b, 0, k, 0.0, c, 0, 1)
    assert c64[0] == 4096.0


def test_similarity_rule_matches_the_reference_margins():
    f = lambda x, y, p=32: oracle.count_mismatches(p, np.array([x]), np.array([y]))[0]
    assert f(1.0, 1.0) == 0
    assert f(1.0, 1.004) == 0          # relative 0.2 % of |x|+|y|
    assert f(1.0, 1.02) == 1           # relative 1 % > 0.5 %
    assert f(0.0, 0.0005) == 0         # one value zero: absolute margin 1e-3
    assert f(0.0, 0.002) == 1
    assert f(np.nan, np.inf) == 0      # both non-finite
    assert f(np.nan, 1.0) == 1
    assert f(1.0, 1.1, 16) == 0        # half: 8 % relative, 0.15 absolute
    assert f(10.0, 12.0, 16) == 1
