"""CPU restatement (numpy + ml_dtypes) of pratchya's FP8 block-quantization path.

TEST INFRASTRUCTURE ONLY.  This module is the parity checker and the timed CPU
baseline.  Nothing in the shipped package imports it; the product path is the
CUDA library and fails loudly without it.

PARITY UNPINNED: the reference ships no tests, fixtures or golden vectors for
this path, and its own implementation (JAX) cannot be imported on this image,
so this restatement is anchored only on the reference's source text and on
known answers derived by hand from its rule (tests/golden/).

Every function cites the reference lines it follows
(paths are relative to the reference project root).

Array conventions (same as the reference):
  value   : float8_e4m3fn, same shape as the input            (_qarr.py:506)
  sc_fp8  : float8_e8m0fnu as raw uint8 bytes, shape [..., M, K]
  sc_fp32 : float32, shape [..., M, 1, 1]
where the input's last two dims are cut into (a, b) blocks numbered row-major,
K = gcd(max(1, a*b//16), #blocks) consecutive blocks form a super-group and
M = #blocks // K.
"""
from __future__ import annotations

import math

import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16
E4M3 = ml_dtypes.float8_e4m3fn
E5M2 = ml_dtypes.float8_e5m2

_OUT_FORMATS = {"e4m3": E4M3, "e5m2": E5M2}


def group_geometry(rows: int, cols: int, tgrid):
    """(M, K) of the scale arrays.  pratchya/_qualia/_qarr.py:474-480."""
    a, b = tgrid
    if rows % a or cols % b:
        raise ValueError(f"shape ({rows},{cols}) not divisible by tgrid {tgrid}")
    m_blocks = (rows * cols) // (a * b)
    target_k = max(1, (a * b) // 16)
    k = math.gcd(target_k, m_blocks)
    return m_blocks // k, k


def _to_blocked(x, a, b, m, k):
    """[..., R, C] -> [..., M, K, a, b].  _qarr.py:470-472, 482."""
    shape = x.shape
    xr = x.reshape(*shape[:-2], shape[-2] // a, a, shape[-1] // b, b)
    nd = xr.ndim
    perm = list(range(nd - 4)) + [nd - 4, nd - 2, nd - 3, nd - 1]
    xr = xr.transpose(*perm)
    return xr.reshape(*shape[:-2], m, k, a, b)


def _from_blocked(xb, shape, a, b):
    """[..., M, K, a, b] -> [..., R, C].  _qarr.py:503-504."""
    xr = xb.reshape(*shape[:-2], shape[-2] // a, shape[-1] // b, a, b)
    nd = xr.ndim
    perm = list(range(nd - 4)) + [nd - 4, nd - 2, nd - 3, nd - 1]
    return xr.transpose(*perm).reshape(*shape)


def _e8m0_to_f32(sc8_u8):
    """byte << 23 reinterpreted as float32 (byte 0 -> 0.0).  _qarr.py:495, 562."""
    return (sc8_u8.astype(np.uint32) << np.uint32(23)).view(np.float32)


def quantize_impl(x, tgrid=(128, 128), out_format: str = "e4m3"):
    """pratchya/_qualia/_qarr.py:458-506.

    `out_format="e5m2"` is not in the reference: it swaps only the final
    bf16 -> fp8 cast (line 499) and keeps every other step.
    """
    x = np.asarray(x)
    orig_shape = x.shape
    if x.ndim == 1:                                   # :461-462
        x = x.reshape(1, orig_shape[0])
    elif x.ndim == 0:                                 # :463-464
        x = x.reshape(1, 1)
    shape = x.shape
    a, b = tgrid
    m, k = group_geometry(shape[-2], shape[-1], tgrid)

    xb = _to_blocked(x, a, b, m, k)
    # :484  block amax (computed in the input dtype, then widened: exact)
    m_i = np.max(np.abs(xb), axis=(-2, -1), keepdims=True).astype(np.float32)
    # :485  super-group amax
    big_m = np.max(m_i, axis=(-3, -2, -1), keepdims=True)
    # :488-489
    safe = np.where(big_m == np.float32(0.0), np.float32(1.0), big_m)
    s_f32 = (m_i / safe).astype(np.float32)
    # :492-493  biased exponent byte == floor-to-power-of-two in e8m0
    sb = (s_f32.view(np.uint32) >> np.uint32(23)).astype(np.uint8)
    # :495-497
    s_q = _e8m0_to_f32(sb)
    s_eff = (s_q * big_m).astype(np.float32)
    s_eff = np.maximum(s_eff, np.float32(1e-7))
    # :499  f32 divide, exact *128, then f32 -> bf16 -> fp8, both round-to-nearest-even
    v = (xb.astype(np.float32) / s_eff) * np.float32(128.0)
    q = v.astype(BF16).astype(_OUT_FORMATS[out_format])
    q = _from_blocked(q, shape, a, b).reshape(orig_shape)          # :503-506
    sc8 = sb.reshape(*shape[:-2], m, k)                            # :500, 506
    sc32 = big_m.reshape(*shape[:-2], m, 1, 1).astype(np.float32)  # :501, 506
    return q, sc8, sc32


def dequantize_impl(x_fp8, sc_fp8, sc_fp32, dtype, tgrid):
    """pratchya/_qualia/_qarr.py:541-569 (no 1e-7 floor on this side)."""
    x_fp8 = np.asarray(x_fp8)
    orig_shape = x_fp8.shape
    if x_fp8.ndim == 1:
        x_fp8 = x_fp8.reshape(1, orig_shape[0])
    elif x_fp8.ndim == 0:
        x_fp8 = x_fp8.reshape(1, 1)
    shape = x_fp8.shape
    m, k = sc_fp8.shape[-2:]                                       # :550
    a, b = tgrid
    xb = _to_blocked(x_fp8, a, b, m, k)
    sc8 = np.asarray(sc_fp8).view(np.uint8).reshape(*shape[:-2], m, k, 1, 1)
    sc32 = np.asarray(sc_fp32, dtype=np.float32).reshape(*shape[:-2], m, 1, 1, 1)
    x_sc = (_e8m0_to_f32(sc8) * sc32).astype(np.float32)           # :562-563
    out = xb.astype(BF16).astype(np.float32) * x_sc / np.float32(128.0)   # :564
    out = _from_blocked(out.astype(np.float32), shape, a, b)
    return out.reshape(orig_shape).astype(dtype)                   # :569


def dequantize_impl_bwd(sc_fp8, sc_fp32, g_out, tgrid):
    """Cotangent of the fp8 value: g * x_sc / 128.  _qarr.py:575-601."""
    g = np.asarray(g_out)
    shape = g.shape
    g32 = g.astype(np.float32)
    if g32.ndim == 1:
        g32 = g32.reshape(1, shape[0])
    elif g32.ndim == 0:
        g32 = g32.reshape(1, 1)
    s2 = g32.shape
    m, k = sc_fp8.shape[-2:]
    a, b = tgrid
    gb = _to_blocked(g32, a, b, m, k)
    sc8 = np.asarray(sc_fp8).view(np.uint8).reshape(*s2[:-2], m, k, 1, 1)
    sc32 = np.asarray(sc_fp32, dtype=np.float32).reshape(*s2[:-2], m, 1, 1, 1)
    x_sc = (_e8m0_to_f32(sc8) * sc32).astype(np.float32)
    gx = (gb * x_sc / np.float32(128.0)).astype(np.float32)
    return _from_blocked(gx, s2, a, b).reshape(shape).astype(g.dtype)


def quantize_impl_bwd(g_triple_or_array, tgrid):
    """_qarr.py:514-526: a non-fp8 cotangent passes through; an fp8 triple is
    dequantized to f32 after NaN e8m0 bytes (0xFF) are replaced by 1.0 (byte 127)."""
    if not isinstance(g_triple_or_array, tuple):
        return g_triple_or_array
    g_fp8, g_sc8, g_sc32 = g_triple_or_array
    if np.asarray(g_fp8).dtype != E4M3:
        return g_fp8
    g_sc8 = np.asarray(g_sc8).view(np.uint8)
    g_sc8 = np.where(g_sc8 == 0xFF, np.uint8(127), g_sc8)
    return dequantize_impl(g_fp8, g_sc8, g_sc32, np.float32, tgrid)


def quantize_nd(x, tgrid, out_format="e4m3"):
    """QArrayImpl.__quantize: a 3-D value is quantized per leading index
    (lax.scan), so super-groups never cross it.  _qarr.py:34-44."""
    x = np.asarray(x)
    if x.ndim == 3:
        parts = [quantize_impl(x[i], tgrid, out_format) for i in range(x.shape[0])]
        return tuple(np.stack([p[j] for p in parts]) for j in range(3))
    return quantize_impl(x, tgrid, out_format)


def dequantize_nd(x_fp8, sc_fp8, sc_fp32, dtype, tgrid):
    """QArrayImpl.dequantize.  _qarr.py:46-59."""
    x_fp8 = np.asarray(x_fp8)
    if x_fp8.ndim == 3:
        return np.stack([dequantize_impl(x_fp8[i], sc_fp8[i], sc_fp32[i], dtype, tgrid)
                         for i in range(x_fp8.shape[0])])
    return dequantize_impl(x_fp8, sc_fp8, sc_fp32, dtype, tgrid)


def adapt_grid(tgrid, shape):
    """gcd grid rule used by _requantize/apply/concat/__getitem__.  _qarr.py:371-380."""
    old_a, old_b = tgrid
    if len(shape) == 0:
        h, w = 1, 1
    elif len(shape) == 1:
        h, w = 1, shape[0]
    else:
        h, w = shape[-2:]
    return (math.gcd(old_a, h), math.gcd(old_b, w))


def matmul_impl(x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32, grid_x, grid_y, acc=np.float32):
    """dq(X) @ dq(Y) in f32.  _qarr.py:605-608.  `acc=np.float64` gives the
    high-precision value GEMM tolerances are measured against."""
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, grid_x)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, grid_y)
    return np.matmul(x.astype(acc), y.astype(acc))


def _reduce_broadcast(g, target_shape):
    """_qarr.py:624-632."""
    if g.shape == tuple(target_shape):
        return g
    axes = list(range(g.ndim - len(target_shape)))
    lead = len(axes)
    for i, (gs, ts) in enumerate(zip(g.shape[lead:], target_shape)):
        if ts == 1 and gs > 1:
            axes.append(lead + i)
    return np.sum(g, axis=tuple(axes)).reshape(target_shape)


def matmul_impl_bwd(res, g_out, grid_x, grid_y):
    """_qarr.py:616-640: f32 dots on dequantized operands, both gradients
    returned as fp8 triples on their operand's grid."""
    x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32 = res
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, grid_x)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, grid_y)
    g = np.asarray(g_out, dtype=np.float32)
    gx = g @ np.swapaxes(y, -1, -2)
    gy = np.swapaxes(x, -1, -2) @ g
    gx = _reduce_broadcast(gx, x_fp8.shape)
    gy = _reduce_broadcast(gy, y_fp8.shape)
    return quantize_impl(gx, grid_x), quantize_impl(gy, grid_y)


def matmul_mixed_impl(x_fp8, x_sc8, x_sc32, y_f32, grid_x):
    """_qarr.py:645-647."""
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, grid_x)
    return np.matmul(x, np.asarray(y_f32, dtype=np.float32))


def rmatmul_mixed_impl(x_f32, y_fp8, y_sc8, y_sc32, grid_y):
    """_qarr.py:680-682."""
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, grid_y)
    return np.matmul(np.asarray(x_f32, dtype=np.float32), y)


_ELEMENTWISE = {
    "add": np.add, "mul": np.multiply, "sub": np.subtract, "truediv": np.divide,
    "floordiv": np.floor_divide, "mod": np.mod, "pow": np.power,
}


def elementwise_impl(op: str, x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32, tgrid):
    """_qarr.py:715-763: dequantize both (same grid), apply op, f32 out."""
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, tgrid)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, tgrid)
    with np.errstate(all="ignore"):
        return _ELEMENTWISE[op](x, y).astype(np.float32)


def fp8_matmul(x_f32, y_f32, tgrid=(1, 16)):
    """_qarr.py:766-771: Q(x,t) @ Q(y,t) -> re-quantized (t[0], t[1]) -> f32."""
    xq = quantize_nd(np.asarray(x_f32, dtype=np.float32), tgrid)
    yq = quantize_nd(np.asarray(y_f32, dtype=np.float32), tgrid)
    out = matmul_impl(*xq, *yq, tgrid, tgrid)
    out_grid = (tgrid[0], tgrid[1])                                 # :105
    oq = quantize_nd(out, out_grid)
    return dequantize_nd(*oq, np.float32, out_grid)


def fp8_matmul_bwd(x_f32, y_f32, g_out, tgrid=(1, 16)):
    """_qarr.py:780-791."""
    y_t = np.swapaxes(np.asarray(y_f32), -1, -2)
    x_t = np.swapaxes(np.asarray(x_f32), -1, -2)
    return fp8_matmul(g_out, y_t, tgrid), fp8_matmul(x_t, g_out, tgrid)


def linear_forward(x, w_triple, w_grid):
    """Linear.__call__: (Q(x,(1,a)) @ W).astype(x.dtype), where the product is
    re-quantized on (1, b) before the cast.  pratchya/_nnx_impl/_module.py:46-50
    and _qarr.py:99-105."""
    a, b = w_grid
    x = np.asarray(x)
    xq = quantize_nd(x.astype(np.float32), (1, a))
    y = matmul_impl(*xq, *w_triple, (1, a), w_grid)
    yq = quantize_nd(y, (1, b))
    return dequantize_nd(*yq, x.dtype, (1, b))


def effective_scale(sc_fp8, sc_fp32):
    """Per-block multiplier dequantize applies: f32(sc8<<23) * sc32 / 128."""
    sc8 = np.asarray(sc_fp8).view(np.uint8)
    sc32 = np.asarray(sc_fp32, dtype=np.float32).reshape(*sc8.shape[:-1], 1)
    return (_e8m0_to_f32(sc8) * sc32 / np.float32(128.0)).astype(np.float32)


def momentum_update(g_triple, m_triple, tgrid, beta1, beta2):
    """The momentum step of the optimizer for a quantized parameter,
    pratchya/_nnx_impl/_optimizer.py:171-205 (the branch where param is a 2-D QArrayImpl):
    g and m are dequantized to f32 (:178-179); c = beta1*m + (1-beta1)*g (:191),
    new_m = beta2*m + (1-beta2)*g (:192) re-quantized on the parameter's grid (:204-205).
    The Python scalars enter as f32 (JAX weak typing): beta and 1.0 - beta, each rounded once.
    Returns (c f32, new_m triple)."""
    g = dequantize_impl(*g_triple, np.float32, tgrid).astype(np.float32)
    m = dequantize_impl(*m_triple, np.float32, tgrid).astype(np.float32)
    b1, c1 = np.float32(beta1), np.float32(1.0 - beta1)
    b2, c2 = np.float32(beta2), np.float32(1.0 - beta2)
    c = (b1 * m + c1 * g).astype(np.float32)
    new_m = (b2 * m + c2 * g).astype(np.float32)
    return c, quantize_impl(new_m, tgrid)



def matmul_mixed_impl_bwd(res, g_out, grid_x):
    """_qarr.py:654-675: gradients of Q @ dense; only the quantized side's is quantized."""
    x_fp8, x_sc8, x_sc32, y_f32 = res
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, grid_x)
    g = np.asarray(g_out, dtype=np.float32)
    gx = _reduce_broadcast(g @ np.swapaxes(np.asarray(y_f32, dtype=np.float32), -1, -2), x_fp8.shape)
    gy = np.swapaxes(x, -1, -2) @ g
    return quantize_impl(gx, grid_x), gy


def rmatmul_mixed_impl_bwd(res, g_out, grid_y):
    """_qarr.py:689-710: gradients of dense @ Q."""
    x_f32, y_fp8, y_sc8, y_sc32 = res
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, grid_y)
    g = np.asarray(g_out, dtype=np.float32)
    gx = g @ np.swapaxes(y, -1, -2)
    gy = _reduce_broadcast(np.swapaxes(np.asarray(x_f32, dtype=np.float32), -1, -2) @ g, y_fp8.shape)
    return gx, quantize_impl(gy, grid_y)


def _elementwise_vjp(op: str, x, y, g):
    """jax.vjp(op, x, y) applied to g (_qarr.py:732-733), restated from JAX's differentiation rules of the
    lax primitives jnp.add / subtract / multiply / divide / floor_divide / mod / power lower to:
    div -> (g / y, (-g * x) * y**-2); floor_divide ends in a rounding (no gradient); mod = rem(x, y)
    (+ y where the signs differ), rem -> (g, -g * sign(x/y) * floor|x/y|); pow -> (g * y * x**(y-1)
    with 0 at y == 0, g * log(x or 1) * x**y)."""
    f = np.float32
    with np.errstate(all="ignore"):
        if op == "add":
            return g, g
        if op == "sub":
            return g, -g
        if op == "mul":
            return (g * y).astype(f), (x * g).astype(f)
        if op == "truediv":
            return (g / y).astype(f), (((-g) * x).astype(f) * (f(1.0) / (y * y).astype(f)).astype(f)).astype(f)
        if op == "floordiv":
            return np.zeros_like(g), np.zeros_like(g)
        if op == "mod":
            q = (x / y).astype(f)
            rem = np.fmod(x, y).astype(f)
            plus = ((rem < 0) != (y < 0)) & (rem != 0)
            gy = ((-g) * (np.sign(q) * np.floor(np.abs(q))).astype(f)).astype(f)
            return g, np.where(plus, (gy + g).astype(f), gy).astype(f)
        if op == "pow":
            ans = np.power(x, y).astype(f)
            jac = np.where(y == 0, f(0.0), (y * np.power(x, (y - f(1.0)).astype(f)).astype(f)).astype(f)).astype(f)
            safe_x = np.where(x == 0, f(1.0), x).astype(f)
            return (g * jac).astype(f), (g * (np.log(safe_x).astype(f) * ans).astype(f)).astype(f)
    raise ValueError(op)


def elementwise_impl_bwd(op: str, res, g_out, tgrid):
    """_qarr.py:727-752: the backward half of an elementwise impl: both gradients as fp8 triples."""
    x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32 = res
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, np.float32, tgrid)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, np.float32, tgrid)
    g = np.asarray(g_out, dtype=np.float32)
    gx, gy = _elementwise_vjp(op, x, y, g)
    full = np.broadcast_shapes(g.shape, x.shape, y.shape)
    gx = _reduce_broadcast(np.broadcast_to(gx, full), x_fp8.shape)
    gy = _reduce_broadcast(np.broadcast_to(gy, full), y_fp8.shape)
    return quantize_impl(np.ascontiguousarray(gx, dtype=np.float32), tgrid), quantize_impl(np.ascontiguousarray(gy, dtype=np.float32), tgrid)


def momentum_update_stacked(g_triple, m_triple, tgrid, beta1, beta2):
    """The momentum step for a stacked (3-D) quantized parameter, pratchya/_nnx_impl/_optimizer.py:108-160:
    per leading index (lax.scan, :144) gradient and momentum are dequantized to bfloat16 (:113-114), blended in
    bfloat16, c = beta1*m + (1-beta1)*g (:123) and new_m = beta2*m + (1-beta2)*g (:124), and new_m is quantized again
    on the parameter's grid (:134; QArrayImpl casts it to f32 first, _qarr.py:29).
    Arithmetic as jax.numpy defines it for bfloat16 arrays and weakly typed Python scalars: the scalars beta and
    1.0 - beta (computed in double) become bfloat16, and every multiply and add rounds its result to bfloat16.
    UNPINNED: XLA is free to keep such intermediates in f32 (xla_allow_excess_precision); the reference ships
    no output that says which.  Returns (c bf16 [L, R, C], new_m triple with leading dim L)."""
    gq, g8, g32 = g_triple
    mq, m8, m32 = m_triple
    cs, parts = [], []
    b1, c1 = BF16(beta1), BF16(1.0 - beta1)
    b2, c2 = BF16(beta2), BF16(1.0 - beta2)
    for i in range(np.asarray(gq).shape[0]):
        g = dequantize_impl(gq[i], g8[i], g32[i], BF16, tgrid)
        m = dequantize_impl(mq[i], m8[i], m32[i], BF16, tgrid)
        c = ((b1 * m).astype(BF16) + (c1 * g).astype(BF16)).astype(BF16)
        new_m = ((b2 * m).astype(BF16) + (c2 * g).astype(BF16)).astype(BF16)
        cs.append(c)
        parts.append(quantize_impl(new_m.astype(np.float32), tgrid))
    return np.stack(cs), tuple(np.stack([p[j] for p in parts]) for j in range(3))
