"""Parity of Convgemm against the oracle's restatement of the reference's host convolution
(test/routines/levelx/xconvgemm.hpp:151-196). Grid after test/correctness/testblas.hpp:146-158: padding {0,1},
dilation {1,2}, kernel {1,3}, output channels {1,6}, stride {1,3}, input channels {1,2}, both kernel modes."""
import itertools

import numpy as np
import pytest

import clblast_b200 as cb
from oracle import cpu_oracle as oracle
from tests import harness as H

pytestmark = pytest.mark.gpu


def check_conv(torch, rng, precision, mode, channels, height, width, kh, kw, pad, stride, dil, num_kernels, batch,
               offs=(0, 0, 0), weight_scale=1.0):
    oh, ow = oracle.conv_output_size(height, width, kh, kw, pad, pad, stride, stride, dil, dil)
    im = H.rand_buffer(rng, precision, offs[0] + batch * channels * height * width + H.CANARY, -1, 1)
    ker = (H.rand_buffer(rng, precision, offs[1] + num_kernels * channels * kh * kw + H.CANARY, -1, 1)
           * np.asarray(weight_scale, dtype=H.NP_OF[precision]))
    res = H.rand_buffer(rng, precision, offs[2] + batch * num_kernels * oh * ow + H.CANARY, -1, 1)
    res_in = res.copy()
    res_in[offs[2]:offs[2] + batch * num_kernels * oh * ow] = np.nan  # beta is 0: the old result must be ignored
    dim, dker, dres = (H.to_device(torch, precision, x) for x in (im, ker, res_in))
    torch.cuda.synchronize()
    st = cb.Convgemm(mode, channels, height, width, kh, kw, pad, pad, stride, stride, dil, dil, num_kernels, batch, dim,
                     offs[0], dker, offs[1], dres, offs[2], precision=precision)
    assert st == cb.StatusCode.kSuccess, st
    got = H.to_host(precision, dres)
    want = oracle.convgemm(precision, mode, channels, height, width, kh, kw, pad, pad, stride, stride, dil, dil,
                           num_kernels, batch, im, offs[0], ker, offs[1], res, offs[2], f64=True)
    mask = np.zeros(res.size, dtype=bool)
    mask[offs[2]:offs[2] + batch * num_kernels * oh * ow] = True
    H.check_against_oracle(precision, got, want, mask, res_in)
    if precision in (32, 64) and cb.last_kernel().startswith("conv_simt"):
        # k runs ascending over (channel, kh, kw) with fused multiply-adds, as in the reference kernel: bit-identical
        typed = np.zeros_like(res)
        oracle.convgemm(precision, mode, channels, height, width, kh, kw, pad, pad, stride, stride, dil, dil,
                        num_kernels, batch, im, offs[0], ker, offs[1], typed, offs[2])
        assert np.array_equal(got[mask].view(np.uint8), typed[mask].view(np.uint8)), "not bit-identical to the oracle"
    return np.abs(got[mask].astype(np.float64) - want[mask]).max()


@pytest.mark.parametrize("precision", (32, 64, 16))
def test_reference_grid(cuda, precision):
    rng = np.random.default_rng(42)
    i = 0
    for mode, pad, dil, ksz, nk, stride, ch in itertools.product((151, 152), (0, 1), (1, 2), (1, 3), (1, 6), (1, 3),
                                                                 (1, 2)):
        hw, batch = ((7, 1), (8, 3), (13, 2))[i % 3]
        check_conv(cuda, rng, precision, mode, ch, hw, hw + i % 2, ksz, ksz, pad, stride, dil, nk, batch,
                   offs=(0, 0, 0) if i % 2 else (10, 10, 10))
        i += 1


@pytest.mark.parametrize("mode", (151, 152))
def test_tensor_core_convolution_path(cuda, mode):
    """Large fp32 convolutions run on the tensor cores (3xTF32, op(A) gathered from the image by the split warps):
    strides, dilations, padding, both kernel modes, ragged pixel / channel / K extents. fp32-level accuracy against the
    fp64 oracle (not bit-identical to the k-ascending order; B200BLAS_SGEMM=ffma selects the CUDA-core kernel)."""
    rng = np.random.default_rng(mode)
    cases = [
        # channels, H, W, kh, kw, pad, stride, dil, num_kernels, batch
        (64, 56, 56, 3, 3, 1, 1, 1, 128, 4),
        (16, 40, 37, 3, 3, 1, 2, 1, 96, 24),     # stride 2, ragged width, Cout below one tile
        (12, 33, 35, 5, 3, 2, 1, 2, 200, 6),     # rectangular kernel, dilation 2, K = 180 (tail), Cout over one tile
        (64, 28, 28, 1, 1, 0, 1, 1, 64, 16),     # pointwise
        (48, 70, 7, 3, 3, 1, 1, 1, 64, 16),      # rows of 7 output pixels: the gather with per-pixel divisions
        (24, 50, 11, 3, 3, 1, 1, 1, 64, 16),     # rows of 11: groups of eight pixels straddle two rows in every phase
        (9, 64, 64, 3, 3, 1, 1, 1, 64, 4),       # K = 81: weight rows that are not a multiple of 16 bytes
    ]
    for ch, h, w, kh, kw, pad, stride, dil, nk, batch in cases:
        oh, ow = oracle.conv_output_size(h, w, kh, kw, pad, pad, stride, stride, dil, dil)
        im = H.rand_buffer(rng, 32, batch * ch * h * w, -1, 1)
        ker = H.rand_buffer(rng, 32, nk * ch * kh * kw, -1, 1)
        res = cuda.full((batch * nk * oh * ow,), float("nan"), device="cuda")
        dim, dker = H.to_device(cuda, 32, im), H.to_device(cuda, 32, ker)
        cuda.cuda.synchronize()
        assert cb.Convgemm(mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, dim, 0, dker, 0, res,
                           0) == cb.StatusCode.kSuccess
        assert cb.last_kernel().startswith("tc_conv"), (cb.last_kernel(), ch, h, w)
        want = oracle.convgemm(32, mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, im, 0, ker, 0,
                               np.zeros(batch * nk * oh * ow, dtype=np.float32), 0, f64=True)
        got = res.cpu().numpy().astype(np.float64)
        bad, worst = oracle.count_mismatches(32, got, want)
        assert bad == 0, (ch, h, w, worst)
        assert worst <= 2.0 ** -20 * ch * kh * kw, (worst, ch * kh * kw)


def test_kernel_larger_than_image_gives_one_output(cuda):
    rng = np.random.default_rng(1)
    check_conv(cuda, rng, 32, 151, 2, 2, 2, 3, 3, 0, 1, 2, 3, 2)


def test_rectangular_kernel_and_wide_image(cuda):
    rng = np.random.default_rng(2)
    for mode in (151, 152):
        oh, ow = oracle.conv_output_size(20, 33, 3, 5, 1, 1, 2, 2, 1, 1)
        assert (oh, ow) == (10, 16)
        im = H.rand_buffer(rng, 32, 2 * 5 * 20 * 33, -1, 1)
        ker = H.rand_buffer(rng, 32, 7 * 5 * 3 * 5, -1, 1)
        res = np.zeros(2 * 7 * oh * ow, dtype=np.float32)
        dim, dker, dres = (H.to_device(cuda, 32, x) for x in (im, ker, res))
        cuda.cuda.synchronize()
        assert cb.Convgemm(mode, 5, 20, 33, 3, 5, 1, 1, 2, 2, 1, 1, 7, 2, dim, 0, dker, 0, dres, 0) == 0
        want = oracle.convgemm(32, mode, 5, 20, 33, 3, 5, 1, 1, 2, 2, 1, 1, 7, 2, im, 0, ker, 0, res, 0, f64=True)
        bad, _ = oracle.count_mismatches(32, dres.cpu().numpy(), want)
        assert bad == 0


def test_config4_convolution_shape(cuda):
    # batch 32, 64 -> 128 channels, 56x56, 3x3, pad 1: checked on 4 of the 32 images against the oracle, then the full
    # batch against per-image calls
    torch = cuda
    rng = np.random.default_rng(3)
    worst = check_conv(torch, rng, 32, 151, 64, 56, 56, 3, 3, 1, 1, 1, 128, 4, weight_scale=0.05)
    assert worst < 1e-4
    g = torch.Generator(device="cuda").manual_seed(0)
    im = torch.rand(32 * 64 * 56 * 56, generator=g, device="cuda") * 2 - 1
    w = torch.randn(128 * 64 * 9, generator=g, device="cuda") * 0.05
    full = torch.full((32 * 128 * 56 * 56,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    assert cb.Convgemm(151, 64, 56, 56, 3, 3, 1, 1, 1, 1, 1, 1, 128, 32, im, 0, w, 0, full, 0) == 0
    full_kernel = cb.last_kernel()
    per = 128 * 56 * 56
    for n in (0, 13, 31):
        one = torch.full((per,), float("nan"), device="cuda")
        torch.cuda.synchronize()
        assert cb.Convgemm(151, 64, 56, 56, 3, 3, 1, 1, 1, 1, 1, 1, 128, 1, im, n * 64 * 56 * 56, w, 0, one, 0) == 0
        if cb.last_kernel() == full_kernel:
            assert torch.equal(one, full[n * per:(n + 1) * per])
        else:  # one image alone is too small for the tensor-core path: same values to fp32 accuracy, not the same bits
            assert torch.allclose(one, full[n * per:(n + 1) * per], atol=2e-5, rtol=0)


@pytest.mark.parametrize("precision", (16, 64))
def test_half_and_double_convolutions_on_the_tensor_core_kernels(cuda, precision):
    """Large half convolutions run as an implicit GEMM on tcgen05 (each thread gathers its pixel's taps into tensor
    memory), double ones as an implicit GEMM on the FP64 mma.sync kernel; both kernel modes, stride, dilation, ragged extents, unaligned buffers, K that is not a
    multiple of 8, more filters than one tile, against the fp64 oracle with the reference's margins."""
    rng = np.random.default_rng(precision)
    cases = [
        # channels, H, W, kh, kw, pad, stride, dil, num_kernels, batch
        (64, 56, 56, 3, 3, 1, 1, 1, 128, 6),
        (16, 40, 37, 3, 3, 1, 2, 1, 96, 40),
        (12, 33, 35, 5, 3, 2, 1, 2, 200, 9),
    ]
    if precision == 16:
        cases += [(64, 28, 28, 1, 1, 0, 1, 1, 64, 16),     # pointwise: one K block per tile
                  (24, 50, 11, 3, 3, 1, 1, 1, 64, 16)]     # narrow rows
    for mode, (ch, h, w, kh, kw, pad, stride, dil, nk, batch) in itertools.product((151, 152), cases):
        oh, ow = oracle.conv_output_size(h, w, kh, kw, pad, pad, stride, stride, dil, dil)
        im = H.rand_buffer(rng, precision, 5 + batch * ch * h * w, -1, 1)
        ker = (H.rand_buffer(rng, precision, 3 + nk * ch * kh * kw, -1, 1) * 0.1).astype(H.NP_OF[precision])
        res = np.full(7 + batch * nk * oh * ow, np.nan, dtype=H.NP_OF[precision])
        dim, dker, dres = (H.to_device(cuda, precision, x) for x in (im, ker, res))
        cuda.cuda.synchronize()
        st = cb.Convgemm(mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, dim, 5, dker, 3, dres, 7,
                         precision=precision)
        assert st == cb.StatusCode.kSuccess
        # half: implicit GEMM with the im2col matrix in tensor memory; double: implicit GEMM on the FP64 mma.sync kernel
        assert cb.last_kernel().startswith("tc_conv_f16" if precision == 16 else "conv_dmma_f64"), cb.last_kernel()
        want = oracle.convgemm(precision, mode, ch, h, w, kh, kw, pad, pad, stride, stride, dil, dil, nk, batch, im, 5, ker,
                               3, np.zeros_like(res), 7, f64=True)
        got = H.to_host(precision, dres)
        assert np.isnan(got[:7].astype(np.float64)).all()          # nothing before the offset was touched
        bad, worst = oracle.count_mismatches(precision, got[7:], want[7:])
        assert bad == 0, (mode, ch, h, w, worst)
        k = ch * kh * kw
        assert worst <= (2e-3 if precision == 16 else 2.0 ** -48 * k), (worst, k)


_TWO_STEP_SCRIPT = r"""
import hashlib
import numpy as np
import torch
import clblast_b200 as cb
g = torch.Generator(device="cuda").manual_seed(9)
for dt in (torch.float16, torch.float64):
    ch, h, w, nk, batch = 32, 40, 37, 96, 24
    im = ((torch.rand(batch * ch * h * w, generator=g, device="cuda") * 2 - 1)).to(dt)
    ker = ((torch.rand(nk * ch * 9, generator=g, device="cuda") * 2 - 1) * 0.1).to(dt)
    res = torch.zeros(batch * nk * h * w, device="cuda", dtype=dt)
    assert cb.Convgemm(151, ch, h, w, 3, 3, 1, 1, 1, 1, 1, 1, nk, batch, im, 0, ker, 0, res, 0) == 0
    torch.cuda.synchronize()
    want = torch.nn.functional.conv2d(im.view(batch, ch, h, w).double(), ker.view(nk, ch, 3, 3).double(), padding=1)
    err = (res.view(batch, nk, h, w).double() - want).abs().max().item()
    print(cb.last_kernel(), err)
"""


def test_two_step_route_on_request(cuda):
    """B200BLAS_CONV=im2col sends half / double convolutions through im2col into scratch and one strided-batched GEMM
    on the tensor-core kernels (the reference's second method, src/routines/levelx/xconvgemm.cpp:96-112); checked
    against a double-precision convolution in a process of its own (the switch is read once)."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, B200BLAS_CONV="im2col", PYTHONPATH=str(root))
    res = subprocess.run([sys.executable, "-c", _TWO_STEP_SCRIPT], capture_output=True, text=True, env=env, cwd=root,
                         timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [line.split() for line in res.stdout.strip().splitlines()]
    assert len(lines) == 2, res.stdout
    assert lines[0][0].startswith("conv_im2col_tc_f16") and float(lines[0][1]) < 2e-2, lines[0]
    assert lines[1][0].startswith("conv_im2col_dmma_f64") and float(lines[1][1]) < 1e-12, lines[1]
