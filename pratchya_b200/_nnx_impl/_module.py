"""The FP8 linear layers of pratchya/_nnx_impl/_module.py (Linear :39-50, LowRankFFN :74-89)
on torch CUDA tensors.  The weight is held as a QArrayImpl on `tgrid`; a call quantizes the
activation on (1, tgrid[0]) and multiplies on the block-scaled tensor-core kernel.
"""
from __future__ import annotations

import math

import torch

from .. import _lib
from .._qualia import _ops
from .._qualia._qarr import QArrayImpl


def lecun_normal(fan_in: int, fan_out: int, *, generator=None, device="cuda", dtype=torch.float32):
    """Truncated-normal fan-in initialiser (flax `lecun_normal`, used at _module.py:41)."""
    std = math.sqrt(1.0 / fan_in) / 0.87962566103423978
    w = torch.empty((fan_in, fan_out), device=device, dtype=torch.float32)
    torch.nn.init.trunc_normal_(w, mean=0.0, std=std, a=-2 * std, b=2 * std, generator=generator)
    return w.to(dtype)


class Linear:
    """`Linear(fan_in, fan_out, tgrid)`: kernel [fan_in, fan_out] quantized on `tgrid`
    (_module.py:40-44).  `__call__` follows :46-50: the product is re-quantized on
    (1, tgrid[1]) and dequantized to x.dtype, so the layer returns dq(q(Y)).
    `matmul(x)` is the same product without that final fake-quantization."""

    def __init__(self, fan_in: int, fan_out: int, tgrid: tuple, *, kernel=None, generator=None,
                 device="cuda", dtype=torch.float32):
        if kernel is None:
            kernel = lecun_normal(fan_in, fan_out, generator=generator, device=device, dtype=dtype)
        self.kernel = kernel if isinstance(kernel, QArrayImpl) else QArrayImpl(kernel, tuple(tgrid))
        self._steps = {}       # (rows, out dtype) -> LinearStep, or None where the fused path does not apply
        self._steps_kernel = self.kernel

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        a, b = self.kernel.tgrid
        if isinstance(x, torch.Tensor) and x.dim() >= 2 and x.is_cuda and self.kernel.get_value().dim() == 2:
            # the same three reference steps with fewer passes: quantize x and multiply (two launches
            # where the fused step applies), then quantize-and-dequantize the f32 product in one
            y = self.matmul(x, out_dtype=torch.float32)
            return _ops.fake_quantize_impl(y, (1, b), x.dtype)
        x_q = QArrayImpl(x, (1, a))
        return (x_q @ self.kernel).astype(x.dtype)

    def matmul(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """dq(Q(x, (1,a))) @ dq(W) accumulated in fp32, returned in `out_dtype` (default x.dtype)."""
        a, _ = self.kernel.tgrid
        k = self.kernel
        step = self._fused_step(x, out_dtype or x.dtype)
        if step is not None:
            out = self._run_step(step, x)
            if out is not None:
                return out[0].reshape(*x.shape[:-1], out[0].shape[-1])
        xq = _ops.quantize_impl(x, (1, a))
        y_t = k.transposed_value() if _ops._tensor_core_eligible(xq[0], k.get_value(), (1, a), k.tgrid) else None
        return _ops.matmul_impl(*xq, k.get_value(), k.sc_fp8, k.sc_fp32, (1, a), k.tgrid, y_fp8_t=y_t,
                                out_dtype=out_dtype or x.dtype)


    def product(self, x: torch.Tensor) -> QArrayImpl:
        """`QArrayImpl(x, (1, a)) @ kernel` as the reference returns it (_qarr.py:99-105): the product
        re-quantized on (1, b), as a QArrayImpl (1 byte per element plus scales instead of a dense array)."""
        a, b = self.kernel.tgrid
        y = self.matmul(x, out_dtype=torch.float32)
        return QArrayImpl(y, (1, b))

    def _fused_step(self, x, out_dtype):
        """The two-launch path (quantizer that also lays out the GEMM's scales, weight prepared once)
        for 2-D-stackable bf16/f32 inputs against a (128,128) weight; None where it does not apply."""
        k = self.kernel
        kk = x.shape[-1] if x.dim() >= 1 else 0
        if (k.tgrid != (128, 128) or x.dim() < 2 or kk == 0 or kk % 1024 != 0 or not x.is_cuda
                or k.get_value().dim() != 2 or k.get_value().shape[1] % 16 != 0
                or out_dtype not in (torch.float32, torch.bfloat16)):
            return None
        if self._steps_kernel is not k:      # the kernel was replaced: its prepared scales are stale
            self._steps, self._steps_kernel = {}, k
        rows = x.numel() // kk
        key = (rows, out_dtype)
        if key not in self._steps:
            self._steps[key] = _ops.LinearStep(k.transposed_value(), k.sc_fp8, k.sc_fp32, rows, out_dtype)
        return self._steps[key]

    def _run_step(self, step, x, **kwargs):
        """Runs the fused step; None (and the step is dropped for good) when the library says that this weight's
        scales do not allow it.  That answer comes from the argument checks, before anything is launched."""
        try:
            return step(x, **kwargs)
        except _lib.PbError as e:
            if e.status != _lib.PB_ERR_UNSUPPORTED:
                raise
            for key, value in list(self._steps.items()):
                if value is step:
                    self._steps[key] = None
            return None


class ChannelMixFFN:
    """The two Linears of ChannelMix with relu^2 between them (pratchya/_nnx_impl/_module.py:231-233,
    246-250): `w_v(relu(w_k(x).astype(f32)) ** 2)`.  The token shift and lerp in front of it (:240-245)
    are the model's glue and stay with the caller.  Where the fused step applies (f32 x, (128,128)
    kernels, widths that are multiples of 1024) the middle -- fake-quantize of the first product,
    relu^2, quantize for the second product -- is one pass; the result has the bits of the literal
    sequence, which is what runs otherwise."""

    def __init__(self, hidden_size: int, intermediate_size: int, blksize: int = 128, *, generator=None,
                 device="cuda", dtype=torch.float32):
        grid = (blksize, blksize)
        self.w_k = Linear(hidden_size, intermediate_size, grid, generator=generator, device=device, dtype=dtype)
        self.w_v = Linear(intermediate_size, hidden_size, grid, generator=generator, device=device, dtype=dtype)

    def literal(self, x: torch.Tensor) -> torch.Tensor:
        k = self.w_k(x).to(torch.float32)
        k = torch.relu(k) ** 2
        return self.w_v(k)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.float32 or x.dim() < 2:
            return self.literal(x)
        rows = x.numel() // x.shape[-1]
        step_k = self.w_k._fused_step(x, torch.float32)
        probe = torch.empty((rows, self.w_v.kernel.shape[0]), dtype=torch.float32, device=x.device) if step_k is not None else None
        step_v = self.w_v._fused_step(probe, torch.float32) if probe is not None else None
        if step_k is None or step_v is None:
            return self.literal(x)
        r1 = self.w_k._run_step(step_k, x)                             # f32 product of the first Linear
        r2 = self.w_v._run_step(step_v, r1[0], relu2_of_fake_quantized=True) if r1 is not None else None     # middle + second product
        if r2 is None:
            return self.literal(x)
        out = _ops.fake_quantize_impl(r2[0], (1, self.w_v.kernel.tgrid[1]), x.dtype)
        return out.reshape(*x.shape[:-1], out.shape[-1])


class LowRankFFN:
    """down (a,1) -> tanh -> up (b,1), _module.py:74-89."""

    def __init__(self, hidden_size: int, lora_rank: int, tgrid: tuple, *, generator=None, device="cuda", dtype=torch.float32):
        a, b = tgrid
        self.down = Linear(hidden_size, lora_rank, (a, 1), generator=generator, device=device, dtype=dtype)
        self.up = Linear(lora_rank, hidden_size, (b, 1), generator=generator, device=device, dtype=dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.up(torch.tanh(self.down(x)))


class _LinearFn(torch.autograd.Function):
    """Differentiable FP8 linear layer: forward and the custom-VJP chain of the reference
    (dequantize_impl_bwd -> quantize_impl_bwd -> matmul_impl_bwd -> quantize_impl_bwd,
    pratchya/_qualia/_qarr.py:575-601, 514-526, 616-640) on the tensor-core kernels.

    recipe "fp8" (default): dY is quantized on (1,128) for dgrad, and both X^T and dY^T are
    quantized on (1,128) along the tokens for wgrad (the operands of fp8_matmul_bwd, :784-789);
    the reference's matmul_impl_bwd keeps dY in f32, which no tensor-core K-block can consume.
    recipe "reference": the literal f32 dots on dequantized operands (library matmul).
    In both, dX is quantized on (1,a) and dequantized again, and dW is quantized on the weight's
    grid, as the reference returns them (:637-640, :522-526)."""

    @staticmethod
    def forward(ctx, x, weight, grid, fake_quant_output, recipe, grad_format, for_backward=True, prepared=None, prepared_x=None):
        a, b = grid
        x2 = x.reshape(-1, x.shape[-1])
        if prepared is not None and "wq" in prepared:
            wq = prepared["wq"]
        else:
            wq = _ops.quantize_impl(weight, grid)
            if prepared is not None:
                prepared["wq"] = wq
        # the tensor-core backward needs the weight as a K-major operand in both directions: (128,128) blocks only.
        # A (128,1) weight (LoRA, gate, lm_head) has one scale per column and 128 rows, which no 128-deep block
        # along its columns can carry: its forward runs on the tensor cores, its backward on the literal recipe.
        want_xt = for_backward and recipe == "fp8" and (a, b) == (128, 128) and x2.shape[0] % 1024 == 0
        if prepared_x is not None:      # x arrives quantized (its producer wrote the triples); x itself is a handle that is not read
            xq, xt = prepared_x
            if a != 128 or xq[0].shape != x2.shape or (want_xt and xt is None):
                raise ValueError("linear_fp8: the quantized input does not fit this layer (grid (1,128), same shape, "
                                 "with its transposed form when a tensor-core backward pass follows)")
        elif want_xt:     # both forms of x in one call (x itself is not kept for the backward pass)
            xq, xt = _ops.quantize_dual_impl(x2)
        else:
            xq, xt = _ops.quantize_impl(x2, (1, a)), None
        eligible = _ops._tensor_core_eligible(xq[0], wq[0], (1, a), grid)
        w_t = None
        if eligible:
            w_t = prepared.get("w_t") if prepared is not None else None
            if w_t is None:
                w_t = _ops.transpose_bytes(wq[0])
                if prepared is not None:
                    prepared["w_t"] = w_t
        y = _ops.matmul_impl(*xq, *wq, (1, a), grid, y_fp8_t=w_t, out_dtype=torch.float32)
        ctx.grid, ctx.recipe, ctx.grad_format, ctx.fake = grid, recipe, grad_format, fake_quant_output
        ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, weight.dtype
        saved = [*xq, *wq]
        if want_xt and eligible:
            saved += list(xt)                                           # X^T on (1,128) for wgrad
            ctx.have_xt = True
        else:
            ctx.have_xt = False
        if fake_quant_output:
            yq = _ops.quantize_impl(y, (1, b))
            y = _ops.dequantize_impl(*yq, x.dtype, (1, b))
            saved += [yq[1], yq[2]]
        else:
            y = y.to(x.dtype)
        ctx.save_for_backward(*saved)
        return y.reshape(*x.shape[:-1], weight.shape[1])

    @staticmethod
    def backward(ctx, g_y):
        a, b = ctx.grid
        saved = list(ctx.saved_tensors)
        xq, wq = saved[0:3], saved[3:6]
        pos = 6
        xt = None
        if ctx.have_xt:
            xt, pos = saved[6:9], 9
        g = g_y.reshape(-1, g_y.shape[-1]).contiguous()
        m, k = xq[0].shape
        n = wq[0].shape[1]
        if ctx.fake and xt is not None and b == 128:
            # the cotangent of the output's dequantize (:575-601) as the prologue of dY's two quantizers
            gq, gt = _ops.dequantize_bwd_quantize_dual_impl(saved[pos], saved[pos + 1], g, out_format=ctx.grad_format)
        else:
            if ctx.fake:                                # cotangent of the output's dequantize, :575-601
                g = _ops.dequantize_impl_bwd(saved[pos], saved[pos + 1], g, (1, b))
            if xt is not None:
                gq, gt = _ops.quantize_dual_impl(g, out_format=ctx.grad_format)
        if xt is not None:
            op = _ops._operand
            gx = _ops.gemm_tn(op(gq[0], gq[1], gq[2], m, n, (1, 128)), op(wq[0], wq[1], wq[2], k, n, (128, 128)), torch.float32, g.device)
            gw = _ops.gemm_tn(op(xt[0], xt[1], xt[2], k, m, (1, 128)), op(gt[0], gt[1], gt[2], n, m, (1, 128)), torch.float32, g.device)
        else:
            x_hat = _ops.dequantize_impl(*xq, torch.float32, (1, a))
            w_hat = _ops.dequantize_impl(*wq, torch.float32, ctx.grid)
            g32 = g.to(torch.float32)
            gx = _ops._matmul_f32(g32, w_hat.t())
            gw = _ops._matmul_f32(x_hat.t(), g32)
        gx = _ops.fake_quantize_impl(gx, (1, a), torch.float32)                                  # :637 then :522-526
        gw = _ops.dequantize_impl(*_ops.quantize_impl(gw, ctx.grid), torch.float32, ctx.grid)    # :638; the optimizer dequantizes it
        return gx.reshape(ctx.x_shape).to(ctx.x_dtype), gw.to(ctx.w_dtype), None, None, None, None, None, None, None


def linear_fp8(x, weight: torch.Tensor, tgrid=(128, 128), *, fake_quant_output: bool = True,
               recipe: str = "fp8", grad_format: str = "e4m3", prepared: dict | None = None) -> torch.Tensor:
    """y = Linear(x) with a dense master `weight` [fan_in, fan_out] that is quantized on `tgrid` in
    the forward pass; differentiable in x and weight.  `grad_format="e5m2"` stores dY in e5m2
    (an extension: the reference has no e5m2 anywhere).  `prepared`: a dict the caller keeps for as long as
    `weight` does not change; the weight's fp8 triple and its byte transpose are put there by the first call and
    reused by the later ones (the passes of one training step quantize the same weight three times otherwise)."""
    if recipe not in ("fp8", "reference"):
        raise ValueError("recipe must be 'fp8' or 'reference'")
    # X^T is quantized in the forward pass only when a backward pass can follow (not under torch.no_grad, as in the first
    # pass of a recomputed block)
    prepared_x = None
    if hasattr(x, "handle"):          # a QuantizedMix: the input's fp8 triples from the kernel that produced it
        x, prepared_x = x.handle, (x.row, x.tokens)
    for_backward = torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad)
    return _LinearFn.apply(x, weight, (int(tgrid[0]), int(tgrid[1])), fake_quant_output, recipe, grad_format, for_backward, prepared, prepared_x)
