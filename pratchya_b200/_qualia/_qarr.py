"""QArrayImpl on torch CUDA tensors: the quantized-array type of
pratchya/_qualia/_qarr.py:15-425 with the same constructor, properties, operators
and grid rules, backed by the sm_100a kernels of libpratchya_b200.so.

A quantized QArrayImpl holds (value fp8 e4m3fn, sc_fp8 e8m0, sc_fp32 f32) + a static
`tgrid`; `QArrayImpl(v, quant=False)` is the reference's unquantized box.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _ops
from ._ops import (E4M3, add_impl, dequantize_impl, floordiv_impl, matmul_impl, matmul_mixed_impl, mod_impl,
                   mul_impl, pow_impl, quantize_impl, rmatmul_mixed_impl, sub_impl, truediv_impl)


def _unwrap_param(other):
    """The reference unwraps nnx.Param-like holders through `.value` (_qarr.py:100-101)."""
    if not isinstance(other, (torch.Tensor, QArrayImpl)) and hasattr(other, "value"):
        return other.value
    return other


def _adapt_grid(tgrid, shape):
    """gcd grid rule, _qarr.py:371-380 (also :272-282, :298-306, :393-401)."""
    old_a, old_b = tgrid
    if len(shape) == 0:
        h, w = 1, 1
    elif len(shape) == 1:
        h, w = 1, shape[0]
    else:
        h, w = shape[-2:]
    return (math.gcd(old_a, h), math.gcd(old_b, w))


class QArrayImpl:
    def __init__(self, value, tgrid: Optional[Tuple[int, int]] = None, quant: bool = True):
        self._value_t = None                       # byte-transposed value, cached for the forward GEMM
        if not quant:                              # _qarr.py:17-18
            self._value = value
        elif isinstance(value, QArrayImpl):        # :20-24
            self._tgrid = value._tgrid
            self._value, self._sc_fp8, self._sc_fp32 = value._value, value._sc_fp8, value._sc_fp32
            self._value_t = value._value_t
        else:                                      # :26-29
            assert tgrid is not None
            self._tgrid = (int(tgrid[0]), int(tgrid[1]))
            self._value, self._sc_fp8, self._sc_fp32 = self._quantize(value)

    # ---- construction helpers ----------------------------------------------------------
    @classmethod
    def from_triple(cls, value, sc_fp8, sc_fp32, tgrid):
        """Rebuilds a QArrayImpl from its leaves (the reference's _tree_unflatten, :413-422)."""
        obj = cls.__new__(cls)
        obj._value_t = None
        obj._tgrid = (int(tgrid[0]), int(tgrid[1]))
        obj._value, obj._sc_fp8, obj._sc_fp32 = value, sc_fp8, sc_fp32
        return obj

    def _is_quantized(self) -> bool:
        return hasattr(self, "_tgrid")

    def get_value(self):
        return self._value

    def _quantize(self, value):
        # Leading dims are quantized slice by slice; for a 3-D value this is the reference's
        # lax.scan over axis 0 (_qarr.py:38-42), and quantize_impl itself batches higher ranks.
        return quantize_impl(value, self._tgrid)

    def dequantize(self, dtype):
        if self._value.dtype != E4M3:              # :47-48
            return self._value.to(dtype)
        return dequantize_impl(self._value, self._sc_fp8, self._sc_fp32, dtype, self._tgrid)

    def __jax_array__(self):                       # name kept from the reference (:61-62)
        return self.dequantize(torch.float32)

    def tree_flatten(self):
        """(children, aux) as the reference registers them with jax (:404-411)."""
        if self._is_quantized():
            return (self._value, self._sc_fp8, self._sc_fp32), (True, self._tgrid)
        return (self._value,), (False, None)

    @classmethod
    def tree_unflatten(cls, aux, children):
        is_quant, tgrid = aux
        if is_quant:
            return cls.from_triple(*children, tgrid)
        return cls(children[0], quant=False)

    # ---- properties ------------------------------------------------------------------------
    @property
    def shape(self):
        return tuple(self._value.shape)

    @property
    def size(self):
        return self._value.numel()

    @property
    def ndim(self):
        return self._value.dim()

    @property
    def dtype(self):
        return self._value.dtype

    @property
    def tgrid(self):
        return self._tgrid

    @property
    def sc_fp8(self):
        return self._sc_fp8

    @property
    def sc_fp32(self):
        return self._sc_fp32

    def transposed_value(self):
        """[N, K] bytes of a 2-D [K, N] value, built once and cached (weights are reused every step)."""
        if self._value_t is None:
            self._value_t = _ops.transpose_bytes(self._value)
        return self._value_t

    # ---- promotion / matmul ------------------------------------------------------------------
    def _promote(self, other, grid_idx=0):         # :80-97
        if isinstance(other, QArrayImpl):
            return other
        other = torch.as_tensor(other, device=self._value.device)
        shape = tuple(other.shape)
        if len(shape) < 2:
            h, w = 1, (shape[0] if len(shape) > 0 else 1)
        else:
            h, w = shape[-2:]
        target_a = self._tgrid[0] if grid_idx == 0 else self._tgrid[1]
        target_b = self._tgrid[1]
        return QArrayImpl(other, tgrid=(math.gcd(target_a, h), math.gcd(target_b, w)))

    def __matmul__(self, other):                   # :99-108
        other = _unwrap_param(other)
        if isinstance(other, QArrayImpl):
            y_t = other._value_t if other._value_t is not None else None
            if y_t is None and _ops._tensor_core_eligible(self._value, other._value, self._tgrid, other._tgrid):
                y_t = other.transposed_value()
            x_out = matmul_impl(self._value, self._sc_fp8, self._sc_fp32, other._value, other._sc_fp8, other._sc_fp32,
                                self._tgrid, other._tgrid, y_fp8_t=y_t)
            return QArrayImpl(x_out, (self._tgrid[0], other._tgrid[1]))
        return matmul_mixed_impl(self._value, self._sc_fp8, self._sc_fp32, other, self._tgrid)

    def __rmatmul__(self, other):                  # :110-119
        other = _unwrap_param(other)
        if isinstance(other, QArrayImpl):
            return other.__matmul__(self)
        return rmatmul_mixed_impl(other, self._value, self._sc_fp8, self._sc_fp32, self._tgrid)

    # ---- elementwise operators (:121-261) ------------------------------------------------------
    def _binary(self, other, impl, op, reflected=False):
        other = _unwrap_param(other)
        if isinstance(other, QArrayImpl):
            lhs, rhs = (other, self) if reflected else (self, other)
            if self._tgrid != other.tgrid:
                return QArrayImpl(op(lhs.astype(torch.float32), rhs.astype(torch.float32)), self._tgrid)
            x_out = impl(lhs._value, lhs._sc_fp8, lhs._sc_fp32, rhs._value, rhs._sc_fp8, rhs._sc_fp32, self._tgrid)
            return QArrayImpl(x_out, self._tgrid)
        mine = self.astype(getattr(other, "dtype", torch.float32) if isinstance(other, torch.Tensor) else torch.float32)
        return op(other, mine) if reflected else op(mine, other)

    def __add__(self, other): return self._binary(other, add_impl, torch.add)
    def __radd__(self, other): return self._binary(other, add_impl, torch.add)          # :132-135 forwards to __add__
    def __sub__(self, other): return self._binary(other, sub_impl, torch.sub)
    def __rsub__(self, other): return self._binary(other, sub_impl, torch.sub, reflected=True)
    def __mul__(self, other): return self._binary(other, mul_impl, torch.mul)
    def __rmul__(self, other): return self._binary(other, mul_impl, torch.mul)          # :170-173 forwards to __mul__
    def __truediv__(self, other): return self._binary(other, truediv_impl, torch.div)
    def __rtruediv__(self, other): return self._binary(other, truediv_impl, torch.div, reflected=True)
    def __floordiv__(self, other): return self._binary(other, floordiv_impl, torch.floor_divide)
    def __rfloordiv__(self, other): return self._binary(other, floordiv_impl, torch.floor_divide, reflected=True)
    def __mod__(self, other): return self._binary(other, mod_impl, torch.remainder)
    def __rmod__(self, other): return self._binary(other, mod_impl, torch.remainder, reflected=True)
    def __pow__(self, other): return self._binary(other, pow_impl, torch.pow)
    def __rpow__(self, other): return self._binary(other, pow_impl, torch.pow, reflected=True)

    # ---- indexing and shape ops ---------------------------------------------------------------
    def __getitem__(self, idx):                    # :263-284
        if not self._is_quantized():
            return QArrayImpl(self.get_value()[idx], quant=False)
        sliced = self.dequantize(torch.float32)[idx]
        return QArrayImpl(sliced, _adapt_grid(self._tgrid, tuple(sliced.shape)))

    def __neg__(self):                             # :286-292: only sc_fp32 changes sign
        return QArrayImpl.from_triple(self._value, self._sc_fp8, -self._sc_fp32, self._tgrid)

    def __abs__(self):                             # :309-315
        v = (self._value.view(torch.uint8) & 0x7F).view(self._value.dtype)
        return QArrayImpl.from_triple(v, self._sc_fp8, self._sc_fp32.abs(), self._tgrid)

    def apply(self, func):                         # :294-307
        out_val = func(self.dequantize(torch.float32))
        return QArrayImpl(out_val, _adapt_grid(self._tgrid, tuple(out_val.shape)))

    def __repr__(self):
        return f"{self._value}"

    @property
    def at(self):                                  # :320-337
        outer = self

        class _Setter:
            def __init__(self, idx):
                self.idx = idx

            def set(self, val):
                val_f32 = val.astype(torch.float32) if isinstance(val, QArrayImpl) else val
                out = outer.dequantize(torch.float32).clone()
                out[self.idx] = val_f32
                return QArrayImpl(out, outer.tgrid)

        class _Helper:
            def __getitem__(self, idx):
                return _Setter(idx)

        return _Helper()

    def astype(self, dtype):                       # :339-342
        if not self._is_quantized():
            return self.get_value().to(dtype)
        return self.dequantize(dtype)

    @property
    def mT(self):                                  # :344-347
        return QArrayImpl(self.astype(torch.float32).mT.contiguous(), (self._tgrid[1], self._tgrid[0]))

    @property
    def T(self):                                   # :349-352
        x = self.astype(torch.float32)
        return QArrayImpl(x.permute(*reversed(range(x.dim()))).contiguous(), (self._tgrid[1], self._tgrid[0]))

    def reshape(self, *args):                      # :354-357
        shape = args[0] if len(args) == 1 and isinstance(args[0], (tuple, list)) else args
        return self._requantize(self.dequantize(torch.float32).reshape(*shape))

    def transpose(self, *axes):                    # :359-363
        axes = axes[0] if len(axes) == 1 and isinstance(axes[0], (tuple, list)) else axes
        x = self.dequantize(torch.float32)
        if len(axes) == 0:
            axes = tuple(reversed(range(x.dim())))
        return self._requantize(x.permute(*axes).contiguous())

    def sum(self, *args, **kwargs):                # :365-368
        if "axis" in kwargs:
            kwargs["dim"] = kwargs.pop("axis")
        if "keepdims" in kwargs:
            kwargs["keepdim"] = kwargs.pop("keepdims")
        return self._requantize(self.dequantize(torch.float32).sum(*args, **kwargs))

    def _requantize(self, out_val):                # :371-380
        return QArrayImpl(out_val, _adapt_grid(self._tgrid, tuple(out_val.shape)))

    @classmethod
    def concat(cls, arrays, axis=0):               # :383-402
        f32 = [a.astype(torch.float32) if isinstance(a, QArrayImpl) else a for a in arrays]
        out = torch.cat(f32, dim=axis)
        first = next((a for a in arrays if isinstance(a, QArrayImpl)), None)
        grid = first.tgrid if first is not None else (1, 128)
        return cls(out, _adapt_grid(grid, tuple(out.shape)))


def _fp8_matmul_value(x_f32, y_f32, tgrid):
    out = QArrayImpl(x_f32, tgrid) @ QArrayImpl(y_f32, tgrid)
    return out.dequantize(torch.float32)


def fp8_matmul_bwd(tgrid, res, g_out):
    """_qarr.py:780-791: both gradients by the same quantized product, on the transposed dense inputs:
    g_x = fp8_matmul(g, y^T), g_y = fp8_matmul(x^T, g)."""
    x_f32, y_f32 = res
    y_t = y_f32.transpose(-1, -2).contiguous()
    x_t = x_f32.transpose(-1, -2).contiguous()
    return _fp8_matmul_value(g_out, y_t, tgrid), _fp8_matmul_value(x_t, g_out, tgrid)


class _Fp8MatmulFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_f32, y_f32, tgrid):
        ctx.save_for_backward(x_f32, y_f32)         # the dense inputs are the residuals (:775-777)
        ctx.tgrid = tgrid
        return _fp8_matmul_value(x_f32, y_f32, tgrid)

    @staticmethod
    def backward(ctx, g_out):
        g_x, g_y = fp8_matmul_bwd(ctx.tgrid, ctx.saved_tensors, g_out.contiguous())
        return g_x, g_y, None


def fp8_matmul(x_f32, y_f32, tgrid=(1, 16)):
    """_qarr.py:766-793: dq(Q(x, t) @ Q(y, t)), differentiable in x and y with the reference's
    custom VJP (fp8_matmul_bwd) instead of the derivative of the forward graph."""
    return _Fp8MatmulFn.apply(x_f32, y_f32, (int(tgrid[0]), int(tgrid[1])))
