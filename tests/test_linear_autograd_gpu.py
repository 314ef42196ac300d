"""The differentiable FP8 linear layer against the oracle's restatement of the reference's VJP chain
(_qarr.py:575-601, 616-640, 514-526).  With recipe="reference" the chain is the reference's own; with
recipe="fp8" (dY and the token-direction operands quantized for the tensor cores) the result is checked
against the oracle run on the same quantized operands, and its deviation from the reference recipe is
only reported.

Every compared quantity has gone through a final fp8 (fake-)quantization of a matmul result.  The
matmuls agree with the oracle's to ~1e-6 (tests/test_gemm_gpu.py), so after that quantization the two
sides are equal to 1e-5 on all but the few elements whose pre-quantization value sits on a rounding
boundary of the cast (or whose block's scale does), and those differ by one fp8 step: the checks below
say exactly that, instead of a blanket 2^-3."""
import numpy as np
import pytest
import torch

from helpers import assert_fake_quantized_close, from_torch, oracle, synth, to_torch
from pratchya_b200._nnx_impl import linear_fp8

pytestmark = pytest.mark.gpu


def reference_chain(x, w, g_y, grid, fake):
    a, b = grid
    xq, wq = oracle.quantize_impl(x, (1, a)), oracle.quantize_impl(w, grid)
    y = oracle.matmul_impl(*xq, *wq, (1, a), grid)
    g = g_y
    if fake:
        yq = oracle.quantize_impl(y, (1, b))
        y = oracle.dequantize_impl(*yq, np.float32, (1, b))
        g = oracle.dequantize_impl_bwd(yq[1], yq[2], g_y, (1, b))
    (gx, gw) = oracle.matmul_impl_bwd((*xq, *wq), g, (1, a), grid)
    return y, oracle.dequantize_impl(*gx, np.float32, (1, a)), oracle.dequantize_impl(*gw, np.float32, grid), g


def rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


@pytest.mark.parametrize("fake", [True, False])
def test_reference_recipe_matches_the_oracle_chain(built_lib, fake):
    m, k, n = 1024, 512, 256
    x, w = synth((m, k), 1), synth((k, n), 2, scale=0.02, outliers=0)
    g_y = synth((m, n), 3, scale=1e-3, outliers=0)
    xt = to_torch(x).requires_grad_(True)
    wt = to_torch(w).requires_grad_(True)
    y = linear_fp8(xt, wt, (128, 128), fake_quant_output=fake, recipe="reference")
    y.backward(to_torch(g_y))
    y_ref, gx_ref, gw_ref, _ = reference_chain(x, w, g_y, (128, 128), fake)
    if fake:
        assert_fake_quantized_close(from_torch(y.detach()), y_ref, "forward")
    else:        # the tensor-core product itself: the GEMM tolerance
        assert rel(from_torch(y.detach()), y_ref) <= 1e-2
    # the cotangent that enters the matmuls is scaled by the output's block scales (:575-601): where the forward's
    # scale bytes differ on a boundary, a whole block of g differs by a factor of two -- rare, and counted below
    assert_fake_quantized_close(from_torch(xt.grad), gx_ref, "dX", boundary_fraction=0.03)
    assert_fake_quantized_close(from_torch(wt.grad), gw_ref, "dW", boundary_fraction=0.03)


@pytest.mark.parametrize("grad_format", ["e4m3", "e5m2"])
def test_fp8_recipe_matches_the_oracle_on_the_same_operands(built_lib, grad_format):
    """dY quantized on (1,128) for dgrad and along the tokens for wgrad, in e4m3 (the reference's dtype) or e5m2
    (the extension): the oracle builds the same operands and multiplies them in f64."""
    m, k, n = 2048, 512, 256
    x, w = synth((m, k), 4), synth((k, n), 5, scale=0.02, outliers=0)
    g_y = synth((m, n), 6, scale=1e-3, outliers=0)
    xt = to_torch(x).requires_grad_(True)
    wt = to_torch(w).requires_grad_(True)
    y = linear_fp8(xt, wt, (128, 128), fake_quant_output=False, recipe="fp8", grad_format=grad_format)
    y.backward(to_torch(g_y))
    wq = oracle.quantize_impl(w, (128, 128))
    w_hat = oracle.dequantize_impl(*wq, np.float64, (128, 128))
    g_hat = oracle.dequantize_impl(*oracle.quantize_impl(g_y, (1, 128), grad_format), np.float64, (1, 128))
    gx = oracle.dequantize_impl(*oracle.quantize_impl((g_hat @ w_hat.T).astype(np.float32), (1, 128)), np.float32, (1, 128))
    xT_hat = oracle.dequantize_impl(*oracle.quantize_impl(np.ascontiguousarray(x.T), (1, 128)), np.float64, (1, 128))
    gT_hat = oracle.dequantize_impl(*oracle.quantize_impl(np.ascontiguousarray(g_y.T), (1, 128), grad_format), np.float64, (1, 128))
    gw = oracle.dequantize_impl(*oracle.quantize_impl((xT_hat @ gT_hat.T).astype(np.float32), (128, 128)), np.float32, (128, 128))
    assert_fake_quantized_close(from_torch(xt.grad), gx, f"dX, dY {grad_format}")
    assert_fake_quantized_close(from_torch(wt.grad), gw, f"dW, dY {grad_format}")
    # deviation of the fp8 recipe from the reference's f32-dY recipe: reported, not bounded
    _, gx_ref, gw_ref, _ = reference_chain(x, w, g_y, (128, 128), False)
    print(f"recipe deviation ({grad_format} dY): dX {rel(from_torch(xt.grad), gx_ref):.3e}, dW {rel(from_torch(wt.grad), gw_ref):.3e}")


def test_batched_bf16_input_with_e5m2_gradients_matches_the_oracle(built_lib):
    """A [2, 512, 256] bf16 activation: leading dims stack into rows, the output is fake-quantized (the layer's
    default), the loss gradient goes back through the output's scales, dY is stored in e5m2."""
    x = synth((2, 512, 256), 7).astype(oracle.BF16)
    w = synth((256, 384), 8, scale=0.02, outliers=0)
    g_y = synth((2, 512, 384), 9, scale=1e-3, outliers=0).astype(oracle.BF16)
    xt = to_torch(x).requires_grad_(True)
    wt = to_torch(w).requires_grad_(True)
    y = linear_fp8(xt, wt, (128, 128), grad_format="e5m2")
    assert y.shape == (2, 512, 384) and y.dtype == torch.bfloat16
    y.backward(to_torch(g_y))
    assert xt.grad.shape == xt.shape and xt.grad.dtype == torch.bfloat16 and wt.grad.shape == wt.shape
    # the oracle on the stacked rows
    x2 = x.astype(np.float32).reshape(1024, 256)
    xq, wq = oracle.quantize_impl(x2, (1, 128)), oracle.quantize_impl(w, (128, 128))
    prod = oracle.matmul_impl(*xq, *wq, (1, 128), (128, 128))
    yq = oracle.quantize_impl(prod, (1, 128))
    y_ref = oracle.dequantize_impl(*yq, oracle.BF16, (1, 128)).reshape(2, 512, 384)
    assert_fake_quantized_close(from_torch(y.detach()).astype(np.float32), y_ref.astype(np.float32), "forward", bf16=True)
    g = oracle.dequantize_impl_bwd(yq[1], yq[2], g_y.reshape(1024, 384), (1, 128)).astype(np.float32)     # stays bf16-valued, as the cotangent's dtype (:599)
    w_hat = oracle.dequantize_impl(*wq, np.float64, (128, 128))
    g_hat = oracle.dequantize_impl(*oracle.quantize_impl(g, (1, 128), "e5m2"), np.float64, (1, 128))
    gx = oracle.dequantize_impl(*oracle.quantize_impl((g_hat @ w_hat.T).astype(np.float32), (1, 128)), np.float32, (1, 128))
    xT_hat = oracle.dequantize_impl(*oracle.quantize_impl(np.ascontiguousarray(x2.T), (1, 128)), np.float64, (1, 128))
    gT_hat = oracle.dequantize_impl(*oracle.quantize_impl(np.ascontiguousarray(g.T), (1, 128), "e5m2"), np.float64, (1, 128))
    gw = oracle.dequantize_impl(*oracle.quantize_impl((xT_hat @ gT_hat.T).astype(np.float32), (128, 128)), np.float32, (128, 128))
    assert_fake_quantized_close(from_torch(xt.grad).astype(np.float32).reshape(1024, 256), gx.astype(oracle.BF16).astype(np.float32), "dX", boundary_fraction=0.03, bf16=True)
    assert_fake_quantized_close(from_torch(wt.grad), gw, "dW", boundary_fraction=0.03)


def test_literal_dot_precision_switch(built_lib):
    """The (128,1)-grid layers' backward dots run on the library matmul: full f32 by default, TF32 operands after
    set_literal_dot_precision("tf32") (what an f32 dot gets on a GPU under XLA's default precision).  TF32 rounds the
    operands to 10 mantissa bits: the gradients move by at most a few 1e-3 of their largest magnitude, and the switch
    changes nothing on the (128,128) tensor-core path."""
    from pratchya_b200._qualia import set_literal_dot_precision
    gen = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(1024, 2048, device="cuda", generator=gen)
    g = torch.randn(1024, 128, device="cuda", generator=gen)
    w = (torch.randn(2048, 128, device="cuda", generator=gen) * 0.02)
    w2 = (torch.randn(2048, 2048, device="cuda", generator=gen) * 0.02)
    g2 = torch.randn(1024, 2048, device="cuda", generator=gen)

    def grads(weight, grid, cot):
        xi, wi = x.clone().requires_grad_(True), weight.clone().requires_grad_(True)
        linear_fp8(xi, wi, grid, fake_quant_output=grid[1] != 1).backward(cot)
        return xi.grad, wi.grad

    try:
        exact = grads(w, (128, 1), g)
        exact_tc = grads(w2, (128, 128), g2)
        set_literal_dot_precision("tf32")
        fast = grads(w, (128, 1), g)
        fast_tc = grads(w2, (128, 128), g2)
    finally:
        set_literal_dot_precision("f32")
    for a, b in zip(exact, fast):
        # both results are re-quantized to fp8 on their way out, so a moved rounding shows as one fp8 step on that element
        diff = (a - b).abs()
        assert diff.mean().item() <= 2e-3 * a.abs().max().item()
    for a, b in zip(exact_tc, fast_tc):
        assert torch.equal(a, b)
    with pytest.raises(ValueError):
        set_literal_dot_precision("bf16")


@pytest.mark.parametrize("rows,cols,fmt", [(1024, 1024, "e4m3"), (4096, 2048, "e5m2"), (32768, 2048, "e4m3"), (8192, 8192, "e4m3")])
def test_output_cotangent_scaling_fused_into_its_quantizers(built_lib, rows, cols, fmt):
    """The first step of a Linear's backward pass: dY through the cotangent rule of the output's dequantize and into its
    two fp8 forms.  The one-call form (the scaling as a prologue of the row quantizer and of the persistent token-major
    quantizer) against the three calls it replaces, byte for byte; fewer tiles than SMs, and many."""
    from pratchya_b200 import _lib
    from pratchya_b200._qualia import _ops, quantize_impl
    gen = torch.Generator(device="cuda").manual_seed(rows + cols)
    y = torch.randn(rows, cols, device="cuda", generator=gen) * 3.0
    y[:, 128:256] *= 1e-3                                        # blocks of very different scale
    y[5] = 0.0                                                   # all-zero super-groups in the output: multiplier zero
    _, y_sc8, y_sc32 = quantize_impl(y, (1, 128))
    g = torch.randn(rows, cols, device="cuda", generator=gen) * 1e-3
    g.view(-1)[::4099] *= 300.0
    got = _ops.dequantize_bwd_quantize_dual_impl(y_sc8, y_sc32, g, out_format=fmt)
    torch.cuda.synchronize()
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    want = _ops.quantize_dual_impl(_ops.dequantize_impl_bwd(y_sc8, y_sc32, g, (1, 128)), out_format=fmt)
    as_bytes = lambda t: t.contiguous().view(torch.uint8)
    for form, a, b in (("row", got[0], want[0]), ("token-major", got[1], want[1])):
        for part, u, v in zip(("fp8", "e8m0", "fp32"), a, b):
            assert u.shape == v.shape and torch.equal(as_bytes(u), as_bytes(v)), f"{form} form, {part}"
