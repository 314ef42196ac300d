"""The FP8 linear layers of pratchya/_nnx_impl/_module.py (Linear :39-50, LowRankFFN :74-89)
on torch CUDA tensors.  The weight is held as a QArrayImpl on `tgrid`; a call quantizes the
activation on (1, tgrid[0]) and multiplies on the block-scaled tensor-core kernel.
"""
from __future__ import annotations

import math

import torch

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

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        a, _ = self.kernel.tgrid
        x_q = QArrayImpl(x, (1, a))
        return (x_q @ self.kernel).astype(x.dtype)

    def matmul(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """dq(Q(x, (1,a))) @ dq(W) accumulated in fp32, returned in `out_dtype` (default x.dtype)."""
        a, _ = self.kernel.tgrid
        k = self.kernel
        xq = _ops.quantize_impl(x, (1, a))
        y_t = k.transposed_value() if _ops._tensor_core_eligible(xq[0], k.get_value(), (1, a), k.tgrid) else None
        return _ops.matmul_impl(*xq, k.get_value(), k.sc_fp8, k.sc_fp32, (1, a), k.tgrid, y_fp8_t=y_t,
                                out_dtype=out_dtype or x.dtype)


class LowRankFFN:
    """down (a,1) -> tanh -> up (b,1), _module.py:74-89."""

    def __init__(self, hidden_size: int, lora_rank: int, tgrid: tuple, *, generator=None, device="cuda", dtype=torch.float32):
        a, b = tgrid
        self.down = Linear(hidden_size, lora_rank, (a, 1), generator=generator, device=device, dtype=dtype)
        self.up = Linear(lora_rank, hidden_size, (b, 1), generator=generator, device=device, dtype=dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.up(torch.tanh(self.down(x)))
