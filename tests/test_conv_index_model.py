"""The index arithmetic of the tensor-memory convolution kernels, restated in numpy and checked against the oracle's
im2col (itself pinned to the reference's im2col kernel source, src/kernels/levelx/im2col.opencl:24-62).

The kernels (clblast_b200/csrc/kernels/gemm_tc_f32_ts.cuh, gemm_tc_f16_conv.cu) decode every K row once per launch
into a table entry {offset of the tap from the pixel's own offset, (kh * dilation) << 16 | kw * dilation}; a gather
thread owns one output pixel, keeps h0 = ho * stride - pad, w0 = wo * stride - pad and pix_off = h0 * W + w0, and loads
image[entry.x + pix_off] when both (unsigned) h0 + dh < H and w0 + dw < W. K rows beyond K get dh = 0x7FFF, pixels
beyond the image h0 = -0x20000000: neither can pass the test. This file checks that recipe, the sentinels included, on
random geometries; it runs on the CPU (the kernels themselves are checked against the oracle on the GPU)."""
import numpy as np
import pytest

from oracle import cpu_oracle as oracle


def tap_table(channels, height, width, kh_n, kw_n, dil_h, dil_w, flip, k_blocks, bk):
    khw = kh_n * kw_n
    k_total = channels * khw
    off = np.zeros(k_blocks * bk, dtype=np.int64)
    packed = np.full(k_blocks * bk, 0x7FFF0000, dtype=np.int64)
    for kg in range(min(k_total, k_blocks * bk)):
        c, k2 = divmod(kg, khw)
        kh, kw = divmod(k2, kw_n)
        if flip:
            kh, kw = kh_n - 1 - kh, kw_n - 1 - kw
        dh, dw = kh * dil_h, kw * dil_w
        off[kg] = (c * height + dh) * width + dw
        packed[kg] = (dh << 16) | dw
    return off, packed


def gathered_matrix(image, channels, height, width, kh_n, kw_n, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w, flip, bk,
                    tile_pixels=128):
    oh, ow = oracle.conv_output_size(height, width, kh_n, kw_n, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w)
    m, k_total = oh * ow, channels * kh_n * kw_n
    k_blocks = -(-k_total // bk)
    off, packed = tap_table(channels, height, width, kh_n, kw_n, dil_h, dil_w, flip, k_blocks, bk)
    tiles = -(-m // tile_pixels)
    pixels = np.arange(tiles * tile_pixels)                      # the last tile runs past the image
    ho, wo = pixels // ow, pixels % ow
    h_first = ho * stride_h - pad_h
    w0 = wo * stride_w - pad_w
    pix_off = h_first * width + w0
    h0 = np.where(pixels < m, h_first, -0x20000000)
    dh, dw = packed >> 16, packed & 0xFFFF
    hh = h0[None, :] + dh[:, None]
    ww = w0[None, :] + dw[:, None]
    inside = (hh >= 0) & (hh < height) & (ww >= 0) & (ww < width)   # the unsigned compares of the kernels
    index = off[:, None] + pix_off[None, :]
    assert index[inside].min(initial=0) >= 0 and index[inside].max(initial=0) < image.size, "a load would leave the image"
    return np.where(inside, image[np.clip(index, 0, image.size - 1)], 0), m, k_total


@pytest.mark.parametrize("bk", (32, 64))
def test_tap_table_and_predicates_reproduce_im2col(bk):
    rng = np.random.default_rng(bk)
    cases = [(3, 9, 11, 3, 3, 1, 1, 1, 1, 1, 1), (5, 20, 7, 5, 3, 2, 0, 2, 1, 1, 2), (2, 6, 6, 1, 1, 0, 0, 1, 1, 1, 1),
             (4, 13, 17, 3, 2, 0, 2, 3, 2, 2, 1), (1, 5, 40, 2, 7, 1, 3, 1, 3, 1, 1), (7, 8, 8, 3, 3, 2, 2, 1, 1, 2, 2)]
    for ch, h, w, kh_n, kw_n, pad_h, pad_w, sh, sw, dh, dw in cases:
        image = rng.standard_normal(ch * h * w).astype(np.float32)
        for mode in (151, 152):
            got, m, k_total = gathered_matrix(image, ch, h, w, kh_n, kw_n, pad_h, pad_w, sh, sw, dh, dw, mode == 152, bk)
            want = oracle.im2col(mode, ch, h, w, kh_n, kw_n, pad_h, pad_w, sh, sw, dh, dw, image, 0,
                                 np.zeros(k_total * m, dtype=np.float32), 0).reshape(k_total, m)
            assert np.array_equal(got[:k_total, :m], want), (ch, h, w, kh_n, kw_n, mode)
            assert not got[k_total:].any(), "K rows of the padding must read as zero"
            assert not got[:, m:].any(), "pixels beyond the image must read as zero"


def test_im2col_kernel_walks_pixels_with_additions_only():
    """im2col_kernel (clblast_b200/csrc/kernels/level3_aux.cu) gives each thread every 256th pixel of a row of the
    column matrix (or one pixel, when several short rows share a CTA) and moves row, column and offset of the tap by
    constants, with one correction when the output column wraps. The same walk in Python must land on the pixels the
    direct formula gives."""
    for height, width in ((56, 56), (7, 7), (20, 33), (300, 5), (5, 300), (17, 16)):
        for k, pad, (sh, sw), (dh_, dw_) in ((1, 0, (1, 1), (1, 1)), (3, 1, (2, 1), (2, 1)), (3, 0, (3, 2), (1, 1)),
                                             (3, 1, (1, 1), (1, 1))):
            oh, ow = oracle.conv_output_size(height, width, k, k, pad, pad, sh, sw, dh_, dw_)
            if oh <= 0 or ow <= 0:
                continue
            plane = oh * ow
            rows_per_cta = 1 if plane >= 256 else 256 // plane
            for kh in range(k):
                for kw in range(k):
                    dh, dw = kh * dh_ - pad, kw * dw_ - pad
                    for tid in range(256):
                        local = tid // plane if rows_per_cta > 1 else 0
                        if local >= rows_per_cta:
                            continue
                        first = tid - local * plane if rows_per_cta > 1 else tid
                        step = plane if rows_per_cta > 1 else 256
                        step_h, step_w = divmod(step, ow)
                        ho0, wo0 = divmod(first, ow)
                        h_step, w_step = step_h * sh, step_w * sw
                        off_step = h_step * width + w_step
                        w_wrap = ow * sw
                        off_wrap = sh * width - w_wrap
                        wo, h, w = wo0, ho0 * sh + dh, wo0 * sw + dw
                        off = h * width + w
                        pos = first
                        while pos < plane:
                            ho_d, wo_d = divmod(pos, ow)
                            assert (h, w, off) == (ho_d * sh + dh, wo_d * sw + dw, (ho_d * sh + dh) * width + wo_d * sw + dw)
                            h, w, off, wo = h + h_step, w + w_step, off + off_step, wo + step_w
                            if wo >= ow:
                                wo, w, h, off = wo - ow, w - w_wrap, h + sh, off + off_wrap
                            pos += step
