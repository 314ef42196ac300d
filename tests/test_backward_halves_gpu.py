"""GPU parity of the backward halves of the quant ops with the oracle's restatement of the reference's
custom VJPs: quantize_impl_bwd (_qarr.py:514-526), matmul_impl_bwd (:616-640), the mixed matmuls
(:654-675, :689-710), the elementwise impls (:727-752) and fp8_matmul_bwd (:780-791).

Where every step is IEEE f32 elementwise arithmetic on bit-identical inputs (quantize_impl_bwd; the
add/sub/mul/div/floor_divide/mod rules) the returned triples are compared bit for bit.  Where an f32
matmul or a transcendental function sits in front of the final quantization its summation order or
last-bit rounding differs between the library and numpy, so a value that lands on a rounding boundary of
the fp8 cast can fall to the other side: there the dequantized results must agree to 1e-5 on all but a
small, stated fraction of elements, and nowhere by more than one fp8 step of the block."""
import numpy as np
import pytest
import torch

from helpers import assert_triple_equal, bytes_of, from_torch, oracle, synth, to_torch
from pratchya_b200._qualia import (add_impl_bwd, dequantize_impl, fp8_matmul, fp8_matmul_bwd, floordiv_impl_bwd,
                                   matmul_impl_bwd, matmul_mixed_impl_bwd, mod_impl_bwd, mul_impl_bwd, pow_impl_bwd,
                                   quantize_impl, quantize_impl_bwd, rmatmul_mixed_impl_bwd, sub_impl_bwd, truediv_impl_bwd)

pytestmark = pytest.mark.gpu


def np_triple(t):
    q, s8, s32 = t
    return (bytes_of(q).view(oracle.E4M3), bytes_of(s8), from_torch(s32))


def assert_quantized_close(got, want, grid, what, boundary_fraction=0.01):
    """Two triples that quantize almost the same f32 array: equal to 1e-5 on all but `boundary_fraction` of the
    elements, and within one fp8 step (2^-3 of the value, 2^-9 of the block's largest representable value for
    small ones) everywhere."""
    a = oracle.dequantize_impl(*np_triple(got), np.float64, grid)
    b = oracle.dequantize_impl(*want, np.float64, grid)
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    scale = np.abs(b).max()
    diff = np.abs(a - b)
    off = diff > 1e-5 * np.abs(b) + 1e-9 * scale
    assert off.mean() <= boundary_fraction, f"{what}: {off.mean():.4f} of the elements differ"
    assert (diff <= 2.0 ** -3 * np.abs(b) + 2.0 ** -9 * scale).all(), f"{what}: a difference exceeds one fp8 step"


def test_quantize_bwd_passes_dense_through_and_repairs_nan_scales(built_lib):
    g = to_torch(synth((64, 256), seed=1))
    assert quantize_impl_bwd(g, (1, 128)) is g                                   # :519-520
    t = quantize_impl(g, (1, 128))
    bad8 = t[1].view(torch.uint8).clone()
    bad8.view(-1)[::5] = 0xFF                                                    # NaN in e8m0
    got = quantize_impl_bwd((t[0], bad8.view(t[1].dtype), t[2]), (1, 128))
    want = oracle.quantize_impl_bwd((bytes_of(t[0]).view(oracle.E4M3), bytes_of(bad8), from_torch(t[2])), (1, 128))
    assert got.dtype == torch.float32
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # an e5m2 cotangent is not e4m3: it passes through as it is
    t5 = quantize_impl(g, (1, 128), out_format="e5m2")
    assert quantize_impl_bwd(t5, (1, 128)) is t5[0]


@pytest.mark.parametrize("gx,gy,shape", [((1, 16), (16, 16), (64, 96, 48)), ((1, 128), (128, 128), (256, 1024, 384)), ((1, 128), (128, 1), (128, 256, 64))])
def test_matmul_bwd_matches_the_oracle(built_lib, gx, gy, shape):
    m, k, n = shape
    x, y = synth((m, k), seed=2), synth((k, n), seed=3, scale=0.02, outliers=0)
    g = synth((m, n), seed=4, scale=1e-3, outliers=0)
    xq, yq = quantize_impl(to_torch(x), gx), quantize_impl(to_torch(y), gy)
    got = matmul_impl_bwd(gx, gy, (*xq, *yq), to_torch(g))
    want_x, want_y = oracle.matmul_impl_bwd((*np_triple(xq), *np_triple(yq)), g, gx, gy)
    assert_quantized_close(got[0:3], want_x, gx, "g_x")
    assert_quantized_close(got[3:6], want_y, gy, "g_y")


def test_matmul_bwd_sums_the_leading_dims_of_a_batched_cotangent(built_lib):
    """reduce_broadcast, :624-635: a [B, M, K] activation against a 2-D weight gives a [B, K, N] weight gradient
    that is summed over B before it is quantized."""
    bsz, m, k, n = 3, 64, 128, 256
    x, y = synth((bsz, m, k), seed=5), synth((k, n), seed=6, scale=0.02, outliers=0)
    g = synth((bsz, m, n), seed=7, scale=1e-3, outliers=0)
    xq, yq = quantize_impl(to_torch(x), (1, 128)), quantize_impl(to_torch(y), (128, 128))
    got = matmul_impl_bwd((1, 128), (128, 128), (*xq, *yq), to_torch(g))
    oxq = oracle.quantize_nd(x, (1, 128))
    x_hat = oracle.dequantize_nd(*oxq, np.float32, (1, 128))
    y_hat = oracle.dequantize_impl(*np_triple(yq), np.float32, (128, 128))
    want_y = oracle.quantize_impl((np.swapaxes(x_hat, -1, -2) @ g).sum(axis=0).astype(np.float32), (128, 128))
    assert tuple(got[3].shape) == (k, n)
    assert_quantized_close(got[3:6], want_y, (128, 128), "g_y summed over the batch")
    want_x = oracle.quantize_nd((g @ y_hat.T).astype(np.float32), (1, 128))
    assert tuple(got[0].shape) == (bsz, m, k)
    for i in range(bsz):
        assert_quantized_close((got[0][i], got[1][i], got[2][i]), tuple(w[i] for w in want_x), (1, 128), f"g_x[{i}]")


def test_mixed_matmul_bwd_matches_the_oracle(built_lib):
    m, k, n = 64, 256, 128
    x, y = synth((m, k), seed=8), synth((k, n), seed=9, scale=0.02, outliers=0)
    g = synth((m, n), seed=10, scale=1e-3, outliers=0)
    xq = quantize_impl(to_torch(x), (1, 128))
    got = matmul_mixed_impl_bwd((1, 128), (*xq, to_torch(y)), to_torch(g))
    want_x, want_gy = oracle.matmul_mixed_impl_bwd((*np_triple(xq), y), g, (1, 128))
    assert_quantized_close(got[0:3], want_x, (1, 128), "Q @ dense: g_x")
    assert np.allclose(got[3].cpu().numpy(), want_gy, rtol=1e-4, atol=1e-6 * np.abs(want_gy).max())
    yq = quantize_impl(to_torch(y), (128, 128))
    got = rmatmul_mixed_impl_bwd((128, 128), (to_torch(x), *yq), to_torch(g))
    want_gx, want_y = oracle.rmatmul_mixed_impl_bwd((x, *np_triple(yq)), g, (128, 128))
    assert np.allclose(got[0].cpu().numpy(), want_gx, rtol=1e-4, atol=1e-6 * np.abs(want_gx).max())
    assert_quantized_close(got[1:4], want_y, (128, 128), "dense @ Q: g_y")


@pytest.mark.parametrize("name,impl_bwd,exact", [("add", add_impl_bwd, True), ("sub", sub_impl_bwd, True), ("mul", mul_impl_bwd, True),
                                                 ("truediv", truediv_impl_bwd, True), ("floordiv", floordiv_impl_bwd, True),
                                                 ("mod", mod_impl_bwd, True), ("pow", pow_impl_bwd, False)])
@pytest.mark.parametrize("grid,shape", [((1, 128), (64, 256)), ((16, 16), (48, 80))])
def test_elementwise_bwd_matches_the_oracle(built_lib, name, impl_bwd, exact, grid, shape):
    x = np.abs(synth(shape, seed=11, outliers=0)) + np.float32(0.25)        # positive base keeps pow and log finite
    y = synth(shape, seed=12, outliers=0) + np.float32(2.5)
    g = synth(shape, seed=13, scale=1e-2, outliers=0)
    xq, yq = quantize_impl(to_torch(x), grid), quantize_impl(to_torch(y), grid)
    got = impl_bwd(grid, (*xq, *yq), to_torch(g))
    want_x, want_y = oracle.elementwise_impl_bwd(name, (*np_triple(xq), *np_triple(yq)), g, grid)
    if exact:
        assert_triple_equal(got[0:3], (want_x[0].view(np.uint8), want_x[1], want_x[2]), f"{name}: g_x")
        assert_triple_equal(got[3:6], (want_y[0].view(np.uint8), want_y[1], want_y[2]), f"{name}: g_y")
    else:
        assert_quantized_close(got[0:3], want_x, grid, f"{name}: g_x")
        assert_quantized_close(got[3:6], want_y, grid, f"{name}: g_y")


@pytest.mark.parametrize("tgrid,shape", [((1, 16), (32, 64, 48)), ((1, 128), (128, 256, 128))])
def test_fp8_matmul_is_differentiable_with_the_reference_vjp(built_lib, tgrid, shape):
    m, k, n = shape
    x, y = synth((m, k), seed=14), synth((k, n), seed=15, scale=0.05, outliers=0)
    g = synth((m, n), seed=16, scale=1e-2, outliers=0)
    xt, yt = to_torch(x).requires_grad_(True), to_torch(y).requires_grad_(True)
    out = fp8_matmul(xt, yt, tgrid)
    out.backward(to_torch(g))
    want_gx, want_gy = oracle.fp8_matmul_bwd(x, y, g, tgrid)

    def close(a, b, what):
        scale = np.abs(b).max()
        diff = np.abs(a.astype(np.float64) - b)
        off = diff > 1e-5 * np.abs(b) + 1e-9 * scale
        assert off.mean() <= 0.02, f"{what}: {off.mean():.4f} of the elements differ"
        assert (diff <= 2.0 ** -3 * np.abs(b) + 2.0 ** -8 * scale).all(), f"{what}: a difference exceeds one fp8 step"

    close(out.detach().cpu().numpy(), oracle.fp8_matmul(x, y, tgrid), "forward")
    close(xt.grad.cpu().numpy(), want_gx, "g_x")
    close(yt.grad.cpu().numpy(), want_gy, "g_y")
    gx2, gy2 = fp8_matmul_bwd(tgrid, (xt.detach(), yt.detach()), to_torch(g))
    assert torch.equal(gx2, xt.grad) and torch.equal(gy2, yt.grad)
