"""JAX bindings of the C ABI: `quantize_impl`, `dequantize_impl` and the forward `matmul_impl`
of pratchya/_qualia/_qarr.py as `jax.ffi.ffi_call` targets.

NOT RUN WHERE THIS PACKAGE IS TESTED: jax is not installed there, so importing this module
raises ImportError.  It is the binding the C ABI was shaped for: build
`pratchya_b200/csrc/xla_ffi_shim.cc` next to a JAX installation (the command is at the top of that
file) and replace the bodies of the reference's three functions with the ones below; the
reference's `custom_vjp` wrappers (:508-528, :571-603, :610-642) keep calling them unchanged.
"""
from __future__ import annotations

import ctypes
import functools
import math
from pathlib import Path

import jax                     # noqa: E402  (ImportError here is the expected outcome without jax)
import jax.numpy as jnp

from . import _lib

_SHIM = Path(__file__).resolve().parent / "csrc" / "libpratchya_b200_xla.so"
_registered = False


def _register():
    global _registered
    if _registered:
        return
    if not _SHIM.exists():
        raise RuntimeError(f"{_SHIM} is missing: build pratchya_b200/csrc/xla_ffi_shim.cc (see the comment at its top)")
    _lib.load()                # libpratchya_b200.so itself, which the shim links against
    shim = ctypes.CDLL(str(_SHIM))
    for target in ("pb_quantize_ffi", "pb_dequantize_ffi", "pb_matmul_ffi"):
        jax.ffi.register_ffi_target(target.replace("_ffi", ""), jax.ffi.pycapsule(getattr(shim, target)), platform="CUDA")
    _registered = True


def _as_2d(shape):
    if len(shape) == 0:
        return (1, 1)
    if len(shape) == 1:
        return (1, shape[0])
    return tuple(shape)


def _geometry(shape, tgrid):
    a, b = tgrid
    rows, cols = shape[-2], shape[-1]
    nb = (rows // a) * (cols // b)
    k = math.gcd(max(1, a * b // 16), nb)
    return nb // k, k, nb


@functools.partial(jax.jit, static_argnames=["tgrid"])
def quantize_impl(x, tgrid=(128, 128)):
    """_qarr.py:458-506."""
    _register()
    shape = _as_2d(x.shape)
    lead = shape[:-2]
    m, k, nb = _geometry(shape, tgrid)
    q, sc8, sc32, _ = jax.ffi.ffi_call("pb_quantize", (
        jax.ShapeDtypeStruct(x.shape, jnp.float8_e4m3fn),
        jax.ShapeDtypeStruct((*lead, m, k), jnp.float8_e8m0fnu),
        jax.ShapeDtypeStruct((*lead, m, 1, 1), jnp.float32),
        jax.ShapeDtypeStruct((max(8 * nb * math.prod(lead), 8),), jnp.uint8),       # pb_quantize_workspace_size
    ))(x, a=tgrid[0], b=tgrid[1])
    return q, sc8, sc32


@functools.partial(jax.jit, static_argnames=["dtype", "tgrid"])
def dequantize_impl(x_fp8, sc_fp8, sc_fp32, dtype, tgrid):
    """_qarr.py:541-569."""
    _register()
    kernel_dtype = dtype if dtype in (jnp.float32, jnp.bfloat16) else jnp.float32
    out = jax.ffi.ffi_call("pb_dequantize", jax.ShapeDtypeStruct(x_fp8.shape, kernel_dtype))(
        x_fp8, sc_fp8, sc_fp32, a=tgrid[0], b=tgrid[1])
    return out.astype(dtype)


@jax.jit
def matmul_impl_forward(x_fp8, x_sc8, x_sc32, w_t_fp8, w_sc8, w_sc32):
    """The product of Linear.__call__ (_module.py:46-50, _qarr.py:605-608) for a (1,128) activation and a
    (128,128) weight whose bytes were transposed once to [N, K] (pb_transpose_bytes); f32 result."""
    _register()
    n = w_t_fp8.shape[0]
    rows = math.prod(x_fp8.shape[:-1])
    depth = x_fp8.shape[-1]
    # an upper bound of pb_gemm_workspace_size: scale-factor atoms and fp32 factors of both operands
    kb = depth // 128
    scratch = 4096 + ((kb + 3) // 4) * 512 * ((rows + 255) // 128 + 2 * ((n + 223) // 224) + 2) + 4 * kb * (rows + n + 1024)
    y, _ = jax.ffi.ffi_call("pb_matmul", (
        jax.ShapeDtypeStruct((*x_fp8.shape[:-1], n), jnp.float32),
        jax.ShapeDtypeStruct((scratch,), jnp.uint8),
    ))(x_fp8, x_sc8, x_sc32, w_t_fp8, w_sc8, w_sc32)
    return y
