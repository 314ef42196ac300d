"""The quantized-momentum step of the reference's optimizer on the CUDA kernels: the branch for 2-D
parameters (pratchya/_nnx_impl/_optimizer.py:171-205, f32 blend) and the scanned branch for stacked 3-D
parameters (:108-160, bfloat16 blend per layer), which is the one the model's scanned blocks take.

Only the part that works on QArrayImpl data is here: the blend of gradient and momentum and the
re-quantization of the new momentum.  What the reference does with `c` afterwards -- sign() for the
Lion branch (:213), Newton-Schulz for the Muon branch (:208) -- and its schedules and parameter
tree handling are the optimizer's own logic and stay with the caller.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .. import _lib
from .._lib import check
from .._qualia._qarr import QArrayImpl


def momentum_update(g: QArrayImpl, m: QArrayImpl, beta1: float, beta2: float):
    """(c, new_m) with c = beta1*dq(m) + (1-beta1)*dq(g) in f32 and new_m = QArrayImpl of
    beta2*dq(m) + (1-beta2)*dq(g) on m's grid, :191-192 and :204-205, in two passes over the bytes."""
    if g.tgrid != m.tgrid or g.shape != m.shape:
        raise ValueError(f"gradient {g.shape} on {g.tgrid} and momentum {m.shape} on {m.tgrid} must match")
    a, b = m.tgrid
    gq, mq = g.get_value().contiguous(), m.get_value().contiguous()
    if gq.dtype != torch.float8_e4m3fn or mq.dtype != torch.float8_e4m3fn:
        raise ValueError("momentum_update works on e4m3 triples")
    shape = tuple(mq.shape)
    shape2 = shape if len(shape) >= 2 else ((1, shape[0]) if len(shape) == 1 else (1, 1))
    rows, cols = shape2[-2], shape2[-1]
    batch = math.prod(shape2[:-2])
    lib = _lib.load()
    dev = mq.device
    g8, g32 = g.sc_fp8.contiguous(), g.sc_fp32.contiguous()
    m8, m32 = m.sc_fp8.contiguous(), m.sc_fp32.contiguous()
    f32 = lambda v: float(np.float32(v))
    with torch.cuda.device(dev):
        c = torch.empty(shape, dtype=torch.float32, device=dev)
        nq = torch.empty(shape, dtype=torch.float8_e4m3fn, device=dev)
        n8 = torch.empty_like(m8)
        n32 = torch.empty_like(m32)
        ws_bytes = lib.pb_momentum_workspace_size(batch, rows, cols, a, b)
        ws = torch.empty(max(ws_bytes, 8), dtype=torch.uint8, device=dev)
        check(lib.pb_momentum_update(gq.data_ptr(), g8.data_ptr(), g32.data_ptr(), mq.data_ptr(), m8.data_ptr(), m32.data_ptr(),
                                     batch, rows, cols, a, b, f32(beta1), f32(1.0 - beta1), f32(beta2), f32(1.0 - beta2),
                                     c.data_ptr(), nq.data_ptr(), n8.data_ptr(), n32.data_ptr(), ws.data_ptr(), ws_bytes,
                                     torch.cuda.current_stream(dev).cuda_stream))
    return c, QArrayImpl.from_triple(nq, n8, n32, (a, b))


def _bf16_scalar(v: float) -> float:
    """A Python scalar as the bfloat16 value it becomes next to a bfloat16 array (weak typing):
    double -> float -> bfloat16, each round-to-nearest-even, returned as a float."""
    bits = int(np.float32(v).view(np.uint32))
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return float(np.uint32(bits).view(np.float32))


def momentum_update_stacked(g: QArrayImpl, m: QArrayImpl, beta1: float, beta2: float):
    """The scanned branch for a stacked parameter [layers, rows, cols], :108-160: per layer g and m are
    dequantized to bfloat16, c = beta1*m + (1-beta1)*g and new_m = beta2*m + (1-beta2)*g are formed in
    bfloat16, and new_m is quantized again on the parameter's grid.  Returns (c bf16, new_m QArrayImpl);
    the update that follows (sign or Newton-Schulz, weight decay, :136-142) stays with the caller."""
    if g.tgrid != m.tgrid or g.shape != m.shape or len(m.shape) != 3:
        raise ValueError(f"gradient {g.shape} on {g.tgrid} and momentum {m.shape} on {m.tgrid} must be equal 3-D stacks")
    a, b = m.tgrid
    gq, mq = g.get_value().contiguous(), m.get_value().contiguous()
    if gq.dtype != torch.float8_e4m3fn or mq.dtype != torch.float8_e4m3fn:
        raise ValueError("momentum_update_stacked works on e4m3 triples")
    layers, rows, cols = mq.shape
    lib = _lib.load()
    dev = mq.device
    g8, g32 = g.sc_fp8.contiguous(), g.sc_fp32.contiguous()
    m8, m32 = m.sc_fp8.contiguous(), m.sc_fp32.contiguous()
    with torch.cuda.device(dev):
        c = torch.empty((layers, rows, cols), dtype=torch.bfloat16, device=dev)
        nq = torch.empty((layers, rows, cols), dtype=torch.float8_e4m3fn, device=dev)
        n8 = torch.empty_like(m8)
        n32 = torch.empty_like(m32)
        ws_bytes = lib.pb_momentum_workspace_size(layers, rows, cols, a, b)
        ws = torch.empty(max(ws_bytes, 8), dtype=torch.uint8, device=dev)
        check(lib.pb_momentum_update_stacked(gq.data_ptr(), g8.data_ptr(), g32.data_ptr(), mq.data_ptr(), m8.data_ptr(), m32.data_ptr(),
                                             layers, rows, cols, a, b, _bf16_scalar(beta1), _bf16_scalar(1.0 - beta1),
                                             _bf16_scalar(beta2), _bf16_scalar(1.0 - beta2),
                                             c.data_ptr(), nq.data_ptr(), n8.data_ptr(), n32.data_ptr(), ws.data_ptr(), ws_bytes,
                                             torch.cuda.current_stream(dev).cuda_stream))
    return c, QArrayImpl.from_triple(nq, n8, n32, (a, b))


def lion_update(c: torch.Tensor, param_f32: torch.Tensor, lr: float, weight_decay: float) -> torch.Tensor:
    """update = -(lr * sign(c) + lr * weight_decay * p), :213-215."""
    return -(lr * torch.sign(c) + lr * weight_decay * param_f32)
