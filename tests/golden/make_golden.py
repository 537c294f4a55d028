"""Generates tests/golden/gemm_cases.npz and conv_cases.npz: small seeded inputs with outputs computed by numpy in
float64 (matrix products by numpy's BLAS, convolutions by explicit patch extraction), independent of the C oracle.

Run from the repository root:  python tests/golden/make_golden.py
"""
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
NP_OF = {16: np.float16, 32: np.float32, 64: np.float64, 3232: np.complex64, 6464: np.complex128}


def rand(rng, precision, size):
    x = rng.uniform(-2, 2, size)
    if precision > 100:
        x = x + 1j * rng.uniform(-2, 2, size)
    return x.astype(NP_OF[precision])


def stored(buf, off, ld, rows, cols, layout):
    """The rows x cols matrix stored at buf[off:] with leading dimension ld, as float64/complex128."""
    r, c = np.arange(rows)[:, None], np.arange(cols)[None, :]
    idx = off + (r * ld + c if layout == 101 else c * ld + r)
    return buf[idx].astype(np.complex128 if np.iscomplexobj(buf) else np.float64)


def gemm_cases():
    rng = np.random.default_rng(20240611)
    out = {}
    n = 0
    for precision in (16, 32, 64, 3232, 6464):
        trs = (111, 112, 113) if precision > 100 else (111, 112)
        for layout in (101, 102):
            for ta in trs:
                for tb in trs:
                    m, nn, k = [(7, 16, 7), (16, 7, 16), (13, 5, 9), (9, 11, 21)][n % 4]
                    ar, ac = (m, k) if ta == 111 else (k, m)
                    br, bc = (k, nn) if tb == 111 else (nn, k)
                    a_ld = (ac if layout == 101 else ar) + n % 3
                    b_ld = (bc if layout == 101 else br) + (n + 1) % 3
                    c_ld = (nn if layout == 101 else m) + (n + 2) % 3
                    a_off, b_off, c_off = (0, 0, 0) if n % 2 else (10, 5, 3)
                    a = rand(rng, precision, a_off + a_ld * (ar if layout == 101 else ac) + 8)
                    b = rand(rng, precision, b_off + b_ld * (br if layout == 101 else bc) + 8)
                    c = rand(rng, precision, c_off + c_ld * (m if layout == 101 else nn) + 8)
                    alpha, beta = [(3.14, 3.14), (1.0, 0.0), (0.7, 0.3)][n % 3]
                    if precision > 100:
                        alpha, beta = alpha + 0.5j, beta - 0.25j
                    A = stored(a, a_off, a_ld, ar, ac, layout)
                    B = stored(b, b_off, b_ld, br, bc, layout)
                    A = A if ta == 111 else (A.T if ta == 112 else A.conj().T)
                    B = B if tb == 111 else (B.T if tb == 112 else B.conj().T)
                    C = alpha * (A @ B) + (beta * stored(c, c_off, c_ld, m, nn, layout) if beta != 0 else 0)
                    key = f"g{n:03d}"
                    out[key + "_meta"] = np.array([precision, layout, ta, tb, m, nn, k, a_off, a_ld, b_off, b_ld, c_off,
                                                   c_ld], dtype=np.int64)
                    out[key + "_scalars"] = np.array([alpha, beta], dtype=np.complex128)
                    out[key + "_a"], out[key + "_b"], out[key + "_c"] = a, b, c
                    out[key + "_want"] = C  # dense m x n, float64 or complex128
                    n += 1
    np.savez_compressed(HERE / "gemm_cases.npz", **out)
    return n


def conv_cases():
    rng = np.random.default_rng(77)
    out = {}
    n = 0
    for mode in (151, 152):
        for (ch, h, w, kh, kw, pad, stride, dil, nk, batch) in [(2, 7, 8, 3, 3, 1, 1, 1, 6, 2), (1, 9, 9, 3, 3, 0, 3, 2, 1, 3),
                                                               (3, 6, 5, 1, 1, 0, 1, 1, 4, 1), (2, 8, 8, 3, 2, 1, 2, 1, 3, 2),
                                                               (2, 2, 2, 3, 3, 0, 1, 2, 3, 2)]:
            size_h, size_w = h + 2 * pad, w + 2 * pad
            ph, pw = dil * (kh - 1) + 1, dil * (kw - 1) + 1
            oh = (size_h - ph) // stride + 1 if size_h >= ph else 1
            ow = (size_w - pw) // stride + 1 if size_w >= pw else 1
            im = rng.uniform(-1, 1, batch * ch * h * w).astype(np.float32)
            ker = rng.uniform(-1, 1, nk * ch * kh * kw).astype(np.float32)
            img = im.reshape(batch, ch, h, w).astype(np.float64)
            wt = ker.reshape(nk, ch, kh, kw).astype(np.float64)
            if mode == 152:
                wt = wt[:, :, ::-1, ::-1]
            res = np.zeros((batch, nk, oh, ow))
            for ho in range(oh):
                for wo in range(ow):
                    for a in range(kh):
                        for b in range(kw):
                            hi, wi = ho * stride - pad + a * dil, wo * stride - pad + b * dil
                            if 0 <= hi < h and 0 <= wi < w:
                                res[:, :, ho, wo] += np.einsum("bc,kc->bk", img[:, :, hi, wi], wt[:, :, a, b])
            key = f"c{n:02d}"
            out[key + "_meta"] = np.array([mode, ch, h, w, kh, kw, pad, stride, dil, nk, batch, oh, ow], dtype=np.int64)
            out[key + "_im"], out[key + "_ker"], out[key + "_want"] = im, ker, res
            n += 1
    np.savez_compressed(HERE / "conv_cases.npz", **out)
    return n


if __name__ == "__main__":
    print("gemm cases:", gemm_cases(), "conv cases:", conv_cases())
