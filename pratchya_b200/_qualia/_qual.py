"""`qx.<name>` dispatcher, pratchya/_qualia/_qual.py:7-57: unbox QArrayImpl arguments
(dequantize to f32), call the array function `<name>`, re-box the result.

The reference resolves `<name>` in jax.numpy, jax.nn, jax.lax (in that order); this
host resolves it in torch, torch.nn.functional, torch.special.
"""
from __future__ import annotations

import torch

from ._qarr import QArrayImpl

_NAMESPACES = (torch, torch.nn.functional, torch.special)


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    for ns in _NAMESPACES:
        if hasattr(ns, name):
            fn = getattr(ns, name)
            break
    else:
        raise AttributeError(f"module '{__name__}' has no attribute '{name}'")

    def wrapper(*args, **kwargs):
        def unwrap(v):
            if isinstance(v, QArrayImpl):
                return v.__jax_array__() if v._is_quantized() else v.get_value()
            return v

        result = fn(*[unwrap(a) for a in args], **{k: unwrap(v) for k, v in kwargs.items()})
        quant_arg = next((a for a in args if isinstance(a, QArrayImpl) and a._is_quantized()), None)

        def rebox(r):
            if quant_arg is not None and tuple(r.shape) == quant_arg.shape:
                return quant_arg._requantize(r)       # same shape: requantize on the gcd grid (:48-49)
            return QArrayImpl(r, quant=False)

        if isinstance(result, tuple):
            return tuple(rebox(r) for r in result)
        return rebox(result)

    return wrapper
