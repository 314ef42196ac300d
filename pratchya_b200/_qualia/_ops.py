"""Functional quant ops on torch CUDA tensors, same names and argument meaning as
pratchya/_qualia/_qarr.py (quantize_impl :459, dequantize_impl :542, matmul_impl :605,
matmul_mixed_impl :645, rmatmul_mixed_impl :680, the seven elementwise impls :757-763).

Every op runs in libpratchya_b200.so on the tensor's device and the current torch
stream.  torch is used for device memory and streams only.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from .. import _lib
from .._lib import PB_BF16, PB_E4M3, PB_E5M2, PB_F32, Operand, check

E4M3 = torch.float8_e4m3fn
E5M2 = torch.float8_e5m2
E8M0 = torch.float8_e8m0fnu
_FMT_CODE = {"e4m3": PB_E4M3, "e5m2": PB_E5M2}
_FMT_DTYPE = {"e4m3": E4M3, "e5m2": E5M2}
_DTYPE_FMT = {E4M3: PB_E4M3, E5M2: PB_E5M2}
_DENSE_CODE = {torch.float32: PB_F32, torch.bfloat16: PB_BF16}


def group_geometry(rows: int, cols: int, tgrid) -> Tuple[int, int]:
    """(M, K) of the scale arrays, _qarr.py:474-480."""
    a, b = tgrid
    if rows % a or cols % b:
        raise ValueError(f"shape ({rows},{cols}) is not divisible by tgrid {tuple(tgrid)}")
    nb = (rows * cols) // (a * b)
    k = math.gcd(max(1, (a * b) // 16), nb)
    return nb // k, k


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(t: torch.Tensor, what: str):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: pratchya_b200 has no CPU path")


def _as_2d(shape):
    """The reference's rank promotion, _qarr.py:460-464."""
    if len(shape) == 0:
        return (1, 1)
    if len(shape) == 1:
        return (1, shape[0])
    return tuple(shape)


def _dense_input(x: torch.Tensor) -> torch.Tensor:
    if x.dtype not in _DENSE_CODE:
        x = x.to(torch.float32)          # QArrayImpl casts to f32 before quantizing, _qarr.py:29
    return x.contiguous()


def quantize_impl(x: torch.Tensor, tgrid=(128, 128), out_format: str = "e4m3"):
    """Block-quantizes the last two dims of `x`; leading dims are independent slices.

    Returns (value fp8 [x.shape], sc_fp8 e8m0 [..., M, K], sc_fp32 f32 [..., M, 1, 1]),
    the triple of _qarr.py:458-506.  `out_format="e5m2"` is an extension that swaps
    only the final cast.
    """
    _require_cuda(x, "quantize_impl input")
    lib = _lib.load()
    orig_shape = tuple(x.shape)
    shape = _as_2d(orig_shape)
    a, b = int(tgrid[0]), int(tgrid[1])
    rows, cols = shape[-2], shape[-1]
    m, k = group_geometry(rows, cols, (a, b))
    lead = shape[:-2]
    batch = math.prod(lead)
    x = _dense_input(x)
    with torch.cuda.device(x.device):
        q = torch.empty(orig_shape, dtype=_FMT_DTYPE[out_format], device=x.device)
        sc8 = torch.empty((*lead, m, k), dtype=E8M0, device=x.device)
        sc32 = torch.empty((*lead, m, 1, 1), dtype=torch.float32, device=x.device)
        if x.numel() == 0:
            return q, sc8, sc32
        ws_bytes = lib.pb_quantize_workspace_size(batch, rows, cols, a, b)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        check(lib.pb_quantize(x.data_ptr(), _DENSE_CODE[x.dtype], batch, rows, cols, a, b, _FMT_CODE[out_format],
                              q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                              ws.data_ptr() if ws is not None else None, ws_bytes, _stream(x)))
    return q, sc8, sc32


def quantize_transposed_impl(x: torch.Tensor, b: int = 128, out_format: str = "e4m3"):
    """The triple of quantize_impl(swapaxes(x, -1, -2), (1, b)) without materialising the
    transpose (the operands fp8_matmul_bwd builds, _qarr.py:784-789)."""
    _require_cuda(x, "quantize_transposed_impl input")
    lib = _lib.load()
    if x.dim() < 2:
        raise ValueError("quantize_transposed_impl needs at least 2 dims")
    rows, cols = x.shape[-2], x.shape[-1]
    lead = tuple(x.shape[:-2])
    batch = math.prod(lead)
    m, k = group_geometry(cols, rows, (1, b))
    x = _dense_input(x)
    with torch.cuda.device(x.device):
        q = torch.empty((*lead, cols, rows), dtype=_FMT_DTYPE[out_format], device=x.device)
        sc8 = torch.empty((*lead, m, k), dtype=E8M0, device=x.device)
        sc32 = torch.empty((*lead, m, 1, 1), dtype=torch.float32, device=x.device)
        if x.numel() == 0:
            return q, sc8, sc32
        ws_bytes = lib.pb_quantize_transposed_workspace_size(batch, rows, cols, b)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=x.device) if ws_bytes else None
        check(lib.pb_quantize_transposed(x.data_ptr(), _DENSE_CODE[x.dtype], batch, rows, cols, b, _FMT_CODE[out_format],
                                         q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                                         ws.data_ptr() if ws is not None else None, ws_bytes, _stream(x)))
    return q, sc8, sc32


def quantize_dual_impl(x: torch.Tensor, out_format: str = "e4m3"):
    """(quantize_impl(x, (1,128)), quantize_transposed_impl(x, 128)) for a 2-D or batched x: the two
    forms a training step needs of an activation or a gradient (_qarr.py:784-789).  One call that
    reads x twice where it applies (bf16, rows % 128 == 0, cols % 1024 == 0), else the two calls."""
    _require_cuda(x, "quantize_dual_impl input")
    if x.dim() < 2:
        raise ValueError("quantize_dual_impl needs at least 2 dims")
    rows, cols = x.shape[-2], x.shape[-1]
    if not (x.dtype == torch.bfloat16 and rows % 128 == 0 and cols % 1024 == 0 and x.numel() > 0):
        return quantize_impl(x, (1, 128), out_format), quantize_transposed_impl(x, 128, out_format)
    lib = _lib.load()
    lead = tuple(x.shape[:-2])
    batch = math.prod(lead)
    m, k = group_geometry(rows, cols, (1, 128))
    mt, kt = group_geometry(cols, rows, (1, 128))
    x = x.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        fmt = _FMT_DTYPE[out_format]
        q = torch.empty(tuple(x.shape), dtype=fmt, device=dev)
        sc8 = torch.empty((*lead, m, k), dtype=E8M0, device=dev)
        sc32 = torch.empty((*lead, m, 1, 1), dtype=torch.float32, device=dev)
        q_t = torch.empty((*lead, cols, rows), dtype=fmt, device=dev)
        sc8_t = torch.empty((*lead, mt, kt), dtype=E8M0, device=dev)
        sc32_t = torch.empty((*lead, mt, 1, 1), dtype=torch.float32, device=dev)
        ws_bytes = lib.pb_quantize_transposed_workspace_size(batch, rows, cols, 128)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        check(lib.pb_quantize_dual(x.data_ptr(), _DENSE_CODE[x.dtype], batch, rows, cols, _FMT_CODE[out_format],
                                   q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), q_t.data_ptr(), sc8_t.data_ptr(), sc32_t.data_ptr(),
                                   ws.data_ptr(), ws_bytes, _stream(x)))
    return (q, sc8, sc32), (q_t, sc8_t, sc32_t)


def dequantize_impl(x_fp8: torch.Tensor, sc_fp8: torch.Tensor, sc_fp32: torch.Tensor, dtype, tgrid):
    """_qarr.py:541-569.  (M, K) come from sc_fp8's last two dims, as in the reference (:550)."""
    _require_cuda(x_fp8, "dequantize_impl input")
    lib = _lib.load()
    orig_shape = tuple(x_fp8.shape)
    shape = _as_2d(orig_shape)
    a, b = int(tgrid[0]), int(tgrid[1])
    rows, cols = shape[-2], shape[-1]
    m, k = group_geometry(rows, cols, (a, b))
    if tuple(sc_fp8.shape[-2:]) != (m, k):
        raise ValueError(f"sc_fp8 has shape {tuple(sc_fp8.shape)}, tgrid {(a, b)} on {shape} needs (..., {m}, {k})")
    batch = math.prod(shape[:-2])
    kernel_dtype = dtype if dtype in _DENSE_CODE else torch.float32
    x_fp8, sc_fp8, sc_fp32 = x_fp8.contiguous(), sc_fp8.contiguous(), sc_fp32.contiguous()
    with torch.cuda.device(x_fp8.device):
        out = torch.empty(orig_shape, dtype=kernel_dtype, device=x_fp8.device)
        if out.numel():
            check(lib.pb_dequantize(x_fp8.data_ptr(), _DTYPE_FMT[x_fp8.dtype], sc_fp8.data_ptr(), sc_fp32.data_ptr(),
                                    batch, rows, cols, a, b, _DENSE_CODE[kernel_dtype], out.data_ptr(), _stream(x_fp8)))
    return out if kernel_dtype == dtype else out.to(dtype)


def fake_quantize_impl(x: torch.Tensor, tgrid, dtype, out_format: str = "e4m3") -> torch.Tensor:
    """dequantize_impl(*quantize_impl(x, tgrid), dtype, tgrid) -- QArrayImpl(x, tgrid).astype(dtype),
    _qarr.py:29 and :339-342 -- in one pass where the library has a fused kernel (f32 input on the
    (1,128) grid with whole 8-block super-groups), otherwise by the two calls.  Same bits either way."""
    _require_cuda(x, "fake_quantize_impl input")
    lib = _lib.load()
    shape = _as_2d(tuple(x.shape))
    a, b = int(tgrid[0]), int(tgrid[1])
    rows, cols = shape[-2], shape[-1]
    fused = (x.dtype == torch.float32 and dtype in _DENSE_CODE and (a, b) == (1, 128) and x.numel() > 0
             and group_geometry(rows, cols, (a, b))[1] == 8)
    if not fused:
        return dequantize_impl(*quantize_impl(x, tgrid, out_format), dtype, tgrid)
    x = x.contiguous()
    with torch.cuda.device(x.device):
        out = torch.empty(tuple(x.shape), dtype=dtype, device=x.device)
        check(lib.pb_fake_quantize(x.data_ptr(), _DENSE_CODE[x.dtype], math.prod(shape[:-2]), rows, cols, a, b,
                                   _FMT_CODE[out_format], out.data_ptr(), _DENSE_CODE[dtype], _stream(x)))
    return out


def relu2_requantize_impl(y: torch.Tensor):
    """quantize_impl(relu(dq(q(y, (1,128))))**2, (1,128)) for an f32 product y [..., cols] with cols % 1024 == 0: the middle
    of ChannelMix between its two Linears (_module.py:246-251: the first Linear's output re-quantization, relu squared, the
    second Linear's input quantization) in one pass over y, with the bits of the three steps run one after another.
    Returns the triple over [rows, cols]."""
    _require_cuda(y, "relu2_requantize_impl input")
    if y.dtype != torch.float32 or y.dim() < 2 or y.shape[-1] % 1024 != 0 or y.numel() == 0:
        raise ValueError(f"relu2_requantize_impl: f32 input with a last dim that is a multiple of 1024, got {y.dtype} {tuple(y.shape)}")
    lib = _lib.load()
    y = y.contiguous()
    cols = y.shape[-1]
    rows = y.numel() // cols
    with torch.cuda.device(y.device):
        q = torch.empty((rows, cols), dtype=E4M3, device=y.device)
        sc8 = torch.empty((rows * cols // 1024, 8), dtype=E8M0, device=y.device)
        sc32 = torch.empty((rows * cols // 1024, 1, 1), dtype=torch.float32, device=y.device)
        check(lib.pb_relu2_requantize(y.data_ptr(), rows, cols, _FMT_CODE["e4m3"], q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                                      None, None, 0, _stream(y)))
    return q, sc8, sc32


def dequantize_impl_bwd(sc_fp8: torch.Tensor, sc_fp32: torch.Tensor, g_out: torch.Tensor, tgrid):
    """Cotangent of the fp8 value: g * x_sc / 128 in g's dtype, _qarr.py:575-601."""
    _require_cuda(g_out, "dequantize_impl_bwd input")
    lib = _lib.load()
    orig_shape = tuple(g_out.shape)
    shape = _as_2d(orig_shape)
    a, b = int(tgrid[0]), int(tgrid[1])
    rows, cols = shape[-2], shape[-1]
    batch = math.prod(shape[:-2])
    g = g_out if g_out.dtype in _DENSE_CODE else g_out.to(torch.float32)
    g = g.contiguous()
    with torch.cuda.device(g.device):
        out = torch.empty_like(g)
        if out.numel():
            check(lib.pb_dequantize_bwd(g.data_ptr(), _DENSE_CODE[g.dtype], sc_fp8.contiguous().data_ptr(),
                                        sc_fp32.contiguous().data_ptr(), batch, rows, cols, a, b, out.data_ptr(), _stream(g)))
    return out.to(g_out.dtype)


def dequantize_bwd_quantize_dual_impl(sc_fp8: torch.Tensor, sc_fp32: torch.Tensor, g_out: torch.Tensor, out_format: str = "e4m3"):
    """quantize_dual_impl(dequantize_impl_bwd(sc_fp8, sc_fp32, g_out, (1,128))): the cotangent of a Linear's fake-quantized output
    through that output's dequantize rule and into the two fp8 forms the layer's backward products take (_qarr.py:575-601, then
    :784-789), in one call that never writes the scaled cotangent.  One call (a row pass and a token-major pass over g_out)
    where it applies (f32, 2-D, rows and cols multiples of 1024); otherwise the two steps.  Same bits either way."""
    _require_cuda(g_out, "dequantize_bwd_quantize_dual_impl input")
    rows, cols = g_out.shape[-2], g_out.shape[-1]
    if not (g_out.dim() == 2 and g_out.dtype == torch.float32 and rows % 1024 == 0 and cols % 1024 == 0 and g_out.numel() > 0):
        return quantize_dual_impl(dequantize_impl_bwd(sc_fp8, sc_fp32, g_out, (1, 128)), out_format=out_format)
    lib = _lib.load()
    g = g_out.contiguous()
    groups = rows * cols // 1024
    dev = g.device
    with torch.cuda.device(dev):
        q = torch.empty((rows, cols), dtype=_FMT_DTYPE[out_format], device=dev)
        sc8 = torch.empty((groups, 8), dtype=E8M0, device=dev)
        sc32 = torch.empty((groups, 1, 1), dtype=torch.float32, device=dev)
        q_t = torch.empty((cols, rows), dtype=_FMT_DTYPE[out_format], device=dev)
        sc8_t = torch.empty((groups, 8), dtype=E8M0, device=dev)
        sc32_t = torch.empty((groups, 1, 1), dtype=torch.float32, device=dev)
        check(lib.pb_dequantize_bwd_quantize_dual(g.data_ptr(), sc_fp8.contiguous().data_ptr(), sc_fp32.contiguous().data_ptr(), rows, cols,
                                                  _FMT_CODE[out_format], q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                                                  q_t.data_ptr(), sc8_t.data_ptr(), sc32_t.data_ptr(), _stream(g)))
    return (q, sc8, sc32), (q_t, sc8_t, sc32_t)


def quantize_impl_bwd(g_out, tgrid):
    """Cotangent rule of quantize_impl, _qarr.py:514-526.  `g_out` is the cotangent of the quantized
    triple: a dense array (any dtype but e4m3) passes through unchanged (:519-520); an e4m3 triple
    (value, sc_fp8, sc_fp32) is dequantized to f32 after the NaN bytes (0xFF) of its e8m0 scales have
    been replaced by 1.0 (byte 127) (:522-526)."""
    if not isinstance(g_out, (tuple, list)):
        return g_out
    g_fp8, g_sc8, g_sc32 = g_out
    if g_fp8.dtype != E4M3:
        return g_fp8
    _require_cuda(g_fp8, "quantize_impl_bwd cotangent")
    b8 = g_sc8.contiguous().view(torch.uint8)
    b8 = torch.where(b8 == 0xFF, torch.full_like(b8, 127), b8).view(E8M0)      # one byte per block: 1/128 of the data
    return dequantize_impl(g_fp8, b8, g_sc32, torch.float32, tgrid)


# ---- matmuls ---------------------------------------------------------------------------

def _tensor_core_eligible(x_fp8, y_fp8, grid_x, grid_y) -> bool:
    """(1,128) activations (any leading dims, 8-block super-groups inside every slice) times a 2-D
    weight on (128,128), or on (128,1) -- the reference's gate, lm_head and LoRA weights
    (pratchya/_nnx_impl/_module.py:82-84, 326): their scales are one e8m0 byte per column and 128-deep
    block, which is a K-major operand with per-row block scales."""
    if x_fp8.dim() < 2 or y_fp8.dim() != 2:
        return False
    mm, kk = x_fp8.shape[-2:]
    k2, nn = y_fp8.shape
    gy = tuple(grid_y)
    if not (tuple(grid_x) == (1, 128) and gy in ((128, 128), (128, 1)) and kk == k2 and kk % 128 == 0 and mm >= 1
            and group_geometry(mm, kk, grid_x)[1] == 8):
        return False
    return nn % 128 == 0 if gy == (128, 128) else nn % 16 == 0


def transpose_bytes(q: torch.Tensor) -> torch.Tensor:
    """[rows, cols] fp8 bytes -> [cols, rows] (a weight prepared for the forward GEMM)."""
    lib = _lib.load()
    rows, cols = q.shape
    q = q.contiguous()
    with torch.cuda.device(q.device):
        out = torch.empty((cols, rows), dtype=q.dtype, device=q.device)
        check(lib.pb_transpose_bytes(q.data_ptr(), rows, cols, out.data_ptr(), _stream(q)))
    return out


def _operand(q, sc8, sc32, rows, depth, grid, transposed_blocks=0) -> Operand:
    return Operand(q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), rows, depth,
                   grid[0], grid[1], _DTYPE_FMT[q.dtype], transposed_blocks)


def gemm_tn(a: Operand, b: Operand, out_dtype, device, keep_alive=()) -> torch.Tensor:
    """D[m, n] = sum_k dq(A)[m, k] * dq(B)[n, k] on the tcgen05 kernel."""
    lib = _lib.load()
    with torch.cuda.device(device):
        d = torch.empty((a.rows, b.rows), dtype=out_dtype, device=device)
        ws_bytes = lib.pb_gemm_workspace_size(a, b)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=device)
        check(lib.pb_gemm_tn(a, b, d.data_ptr(), _DENSE_CODE[out_dtype], b.rows, ws.data_ptr(), ws_bytes,
                             torch.cuda.current_stream(device).cuda_stream))
    return d


GEMM_A_PREPARED = 1
GEMM_B_PREPARED = 2


class LinearStep:
    """quantize(x, (1,128)) followed by dq(x) @ dq(W) for one fixed weight and batch size.

    The two calls of Linear.__call__ (_module.py:46-50) with the per-call re-tiling of the scales
    taken out: the quantizer writes the activation's scales in the GEMM's layout as it goes
    (pb_quantize_for_gemm), and the weight's are prepared by the first call and reused until
    `refresh_weight()` says that its scales changed.  Two launches per call instead of four.

    `w_t` is the byte-transposed fp8 weight [n, k]; `w_sc8`/`w_sc32` its scales from quantizing
    the stored [k, n] matrix on (128,128).  Results are bit-identical to quantize_impl + matmul_impl.
    """

    def __init__(self, w_t, w_sc8, w_sc32, rows: int, out_dtype=torch.bfloat16, out_format: str = "e4m3"):
        _require_cuda(w_t, "LinearStep weight")
        self.n, self.k = int(w_t.shape[0]), int(w_t.shape[1])
        self.rows, self.out_dtype, self.out_format = int(rows), out_dtype, out_format
        if self.k % 1024 != 0:
            raise ValueError(f"LinearStep needs a contraction length that is a multiple of 1024, got {self.k}")
        self._keep = (w_t, w_sc8.contiguous(), w_sc32.contiguous())
        self.b = _operand(w_t, self._keep[1], self._keep[2], self.n, self.k, (128, 128), transposed_blocks=1)
        lib = _lib.load()
        dev = w_t.device
        with torch.cuda.device(dev):
            # the workspace size depends on the shapes and grids only: a placeholder A describes them
            ph = torch.empty(16, dtype=torch.uint8, device=dev)
            a = Operand(ph.data_ptr(), ph.data_ptr(), ph.data_ptr(), self.rows, self.k, 1, 128, _FMT_CODE[out_format], 0)
            self.ws_bytes = lib.pb_gemm_workspace_size(a, self.b)
            if self.ws_bytes == 0:
                raise _lib.PbError(2, lib.pb_last_error().decode(errors="replace"))
            self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self._b_ready = False

    def refresh_weight(self):
        """The weight's scales changed (an optimizer step re-quantized it): prepare them again next call."""
        self._b_ready = False

    def __call__(self, x: torch.Tensor, out=None, triple=None, relu2_of_fake_quantized: bool = False):
        """`relu2_of_fake_quantized`: x is the f32 product of a previous Linear, and this layer's input
        is relu(dq(q(x, (1,128))))**2 (the middle of ChannelMix, _module.py:246-251), computed and
        quantized in the same pass."""
        lib = _lib.load()
        x = _dense_input(x)
        if relu2_of_fake_quantized and x.dtype != torch.float32:
            raise ValueError("relu2_of_fake_quantized needs the f32 product of the previous layer")
        if x.numel() != self.rows * self.k or x.shape[-1] != self.k:
            raise ValueError(f"LinearStep was planned for [{self.rows}, {self.k}], got {tuple(x.shape)}")
        dev = x.device
        with torch.cuda.device(dev):
            if triple is None:
                q = torch.empty((self.rows, self.k), dtype=_FMT_DTYPE[self.out_format], device=dev)
                sc8 = torch.empty((self.rows * self.k // 1024, 8), dtype=E8M0, device=dev)
                sc32 = torch.empty((self.rows * self.k // 1024, 1, 1), dtype=torch.float32, device=dev)
            else:
                q, sc8, sc32 = triple
            d = out if out is not None else torch.empty((self.rows, self.n), dtype=self.out_dtype, device=dev)
            st = torch.cuda.current_stream(dev).cuda_stream
            if relu2_of_fake_quantized:
                check(lib.pb_relu2_requantize(x.data_ptr(), self.rows, self.k, _FMT_CODE[self.out_format],
                                              q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), self.b,
                                              self.ws.data_ptr(), self.ws_bytes, st))
            else:
                check(lib.pb_quantize_for_gemm(x.data_ptr(), _DENSE_CODE[x.dtype], self.rows, self.k, _FMT_CODE[self.out_format],
                                               q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), self.b,
                                               self.ws.data_ptr(), self.ws_bytes, st))
            a = _operand(q, sc8, sc32, self.rows, self.k, (1, 128))
            flags = GEMM_A_PREPARED | (GEMM_B_PREPARED if self._b_ready else 0)
            check(lib.pb_gemm_tn_ex(a, self.b, d.data_ptr(), _DENSE_CODE[self.out_dtype], self.n,
                                    self.ws.data_ptr(), self.ws_bytes, flags, st))
            self._b_ready = True
        return d, (q, sc8, sc32)


def matmul_impl(x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32, block_grid_x, block_grid_y,
                y_fp8_t=None, out_dtype=torch.float32):
    """dq(X) @ dq(Y) with fp32 accumulation, _qarr.py:605-608.

    (1,128) x (128,128) operands run on the block-scaled tcgen05 kernel (`y_fp8_t`, the
    byte-transposed weight, is built here when the caller has not cached it).  Other
    grids follow the reference literally: dequantize both, then an fp32 matmul.
    """
    _require_cuda(x_fp8, "matmul_impl input")
    if _tensor_core_eligible(x_fp8, y_fp8, block_grid_x, block_grid_y):
        lead = tuple(x_fp8.shape[:-2])
        kk = x_fp8.shape[-1]
        mm = x_fp8.numel() // kk          # leading slices stack into rows: their super-groups are 8 blocks each
        nn = y_fp8.shape[1]
        if y_fp8_t is None:
            y_fp8_t = transpose_bytes(y_fp8)
        x_fp8, x_sc8, x_sc32 = x_fp8.contiguous(), x_sc8.contiguous(), x_sc32.contiguous()
        y_sc8, y_sc32 = y_sc8.contiguous(), y_sc32.contiguous()
        a = _operand(x_fp8, x_sc8, x_sc32, mm, kk, (1, 128))
        # the weight's scales were produced on its stored [K, N] view: blocks (128, 128) or (128, 1) there
        b = _operand(y_fp8_t, y_sc8, y_sc32, nn, kk, (block_grid_y[1], 128), transposed_blocks=1)
        d = gemm_tn(a, b, out_dtype, x_fp8.device)
        return d.reshape(*lead, x_fp8.shape[-2], nn) if lead else d
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, block_grid_x)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, block_grid_y)
    return _matmul_f32(x, y).to(out_dtype)


_LITERAL_DOT_TF32 = False


def set_literal_dot_precision(precision: str) -> None:
    """Precision of the library f32 matmul behind the grids the block-scaled kernel cannot take (the reference's
    literal recipe there: dequantize, then an f32 dot).  "f32" (default) keeps full f32 products; "tf32" lets the
    library round the operands to 10 mantissa bits, which is what an f32 dot gets on a GPU under XLA's default
    precision, and is several times faster."""
    global _LITERAL_DOT_TF32
    if precision not in ("f32", "tf32"):
        raise ValueError(f"precision must be 'f32' or 'tf32', got {precision!r}")
    _LITERAL_DOT_TF32 = precision == "tf32"


def _matmul_f32(x, y):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = _LITERAL_DOT_TF32
    try:
        return torch.matmul(x, y)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def matmul_mixed_impl(x_fp8, x_sc8, x_sc32, y_f32, block_grid_x):
    """_qarr.py:645-647."""
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, block_grid_x)
    return _matmul_f32(x, y_f32.to(torch.float32))


def rmatmul_mixed_impl(x_f32, y_fp8, y_sc8, y_sc32, block_grid_y):
    """_qarr.py:680-682."""
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, block_grid_y)
    return _matmul_f32(x_f32.to(torch.float32), y)


def reduce_broadcast(g: torch.Tensor, target_shape) -> torch.Tensor:
    """_qarr.py:624-632: sums the leading dims `g` has on top of `target_shape`, and the dims where the
    target has extent 1, then reshapes to the target."""
    target_shape = tuple(target_shape)
    if tuple(g.shape) == target_shape:
        return g
    lead = g.dim() - len(target_shape)
    axes = list(range(lead))
    for i, (gs, ts) in enumerate(zip(g.shape[lead:], target_shape)):
        if ts == 1 and gs > 1:
            axes.append(lead + i)
    return g.sum(dim=tuple(axes)).reshape(target_shape) if axes else g.reshape(target_shape)


def matmul_impl_bwd(block_grid_x, block_grid_y, res, g_out):
    """_qarr.py:616-640: with the saved triples dequantized, g_x = g @ y^T and g_y = x^T @ g as f32
    dots (the cotangent `g_out` is dense here, so this is the reference's literal recipe on a library
    f32 matmul; the tensor-core recipe that quantizes g is `linear_fp8` / `fp8_matmul_bwd`), leading
    dims reduced, both results returned as fp8 triples on their operand's grid."""
    x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32 = res
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, block_grid_x)
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, block_grid_y)
    g = g_out.to(torch.float32)
    g_x = reduce_broadcast(_matmul_f32(g, y.transpose(-1, -2)), x_fp8.shape)
    g_y = reduce_broadcast(_matmul_f32(x.transpose(-1, -2), g), y_fp8.shape)
    return (*quantize_impl(g_x, block_grid_x), *quantize_impl(g_y, block_grid_y))


def matmul_mixed_impl_bwd(block_grid_x, res, g_out):
    """_qarr.py:654-675: only the quantized side's gradient is quantized."""
    x_fp8, x_sc8, x_sc32, y_f32 = res
    x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, block_grid_x)
    g = g_out.to(torch.float32)
    g_x = reduce_broadcast(_matmul_f32(g, y_f32.to(torch.float32).transpose(-1, -2)), x_fp8.shape)
    g_y = _matmul_f32(x.transpose(-1, -2), g)
    return (*quantize_impl(g_x, block_grid_x), g_y)


def rmatmul_mixed_impl_bwd(block_grid_y, res, g_out):
    """_qarr.py:689-710."""
    x_f32, y_fp8, y_sc8, y_sc32 = res
    y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, block_grid_y)
    g = g_out.to(torch.float32)
    g_x = _matmul_f32(g, y.transpose(-1, -2))
    g_y = reduce_broadcast(_matmul_f32(x_f32.to(torch.float32).transpose(-1, -2), g), y_fp8.shape)
    return (g_x, *quantize_impl(g_y, block_grid_y))


def _elementwise_vjp(op, x, y, g):
    """(g_x, g_y) of op(x, y) under JAX's differentiation rules for the lax primitives the
    reference's jnp functions lower to (jax.vjp(op, x, y) at _qarr.py:732-733), in f32."""
    if op is torch.add:
        return g, g
    if op is torch.sub:
        return g, -g
    if op is torch.mul:
        return g * y, x * g
    if op is torch.div:                   # div: g / y and (-g * x) * y**-2
        return g / y, ((-g) * x) * (1.0 / (y * y))
    if op is torch.floor_divide:          # ends in a rounding: no gradient flows
        return torch.zeros_like(g), torch.zeros_like(g)
    if op is torch.remainder:             # rem(x, y), plus y where the signs differ
        q = x / y
        rem = torch.fmod(x, y)
        plus = ((rem < 0) != (y < 0)) & (rem != 0)
        g_y = (-g) * (torch.sign(q) * torch.floor(torch.abs(q)))
        return g, torch.where(plus, g_y + g, g_y)
    if op is torch.pow:
        ans = torch.pow(x, y)
        jac = torch.where(y == 0, torch.zeros_like(y), y * torch.pow(x, y - 1.0))
        safe_x = torch.where(x == 0, torch.ones_like(x), x)
        return g * jac, g * (torch.log(safe_x) * ans)
    raise ValueError(f"no differentiation rule for {op}")


def make_elementwise_impl_bwd(op):
    """The backward half of make_elementwise_impl, _qarr.py:727-752: dequantize the saved operands,
    pull the cotangent back through `op`, reduce broadcast dims, and return both gradients as fp8
    triples on `tgrid`."""
    def impl_bwd(tgrid, res, g_out):
        x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32 = res
        x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, tgrid)
        y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, tgrid)
        g_x, g_y = _elementwise_vjp(op, x, y, g_out.to(torch.float32))
        g_x = reduce_broadcast(g_x.expand(torch.broadcast_shapes(g_x.shape, x.shape, y.shape)), x_fp8.shape)
        g_y = reduce_broadcast(g_y.expand(torch.broadcast_shapes(g_y.shape, x.shape, y.shape)), y_fp8.shape)
        return (*quantize_impl(g_x.contiguous(), tgrid), *quantize_impl(g_y.contiguous(), tgrid))
    return impl_bwd


_FUSED_OPS = {torch.add: 0, torch.sub: 1, torch.mul: 2, torch.div: 3}


def make_elementwise_impl(op):
    """_qarr.py:715-720: dequantize both operands on the same grid, apply `op`, f32 out.
    add, sub, mul and div of same-shape operands run as one kernel (pb_elementwise, same bits);
    floor_divide, remainder and pow, and broadcasting operands, take the literal three steps."""
    def impl(x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32, tgrid):
        code = _FUSED_OPS.get(op)
        if (code is not None and tuple(x_fp8.shape) == tuple(y_fp8.shape) and x_fp8.numel() > 0
                and tuple(x_sc8.shape) == tuple(y_sc8.shape) and x_fp8.dtype in _DTYPE_FMT and y_fp8.dtype in _DTYPE_FMT):
            _require_cuda(x_fp8, "elementwise input")
            lib = _lib.load()
            shape = _as_2d(tuple(x_fp8.shape))
            a, b = int(tgrid[0]), int(tgrid[1])
            xs = [t.contiguous() for t in (x_fp8, x_sc8, x_sc32, y_fp8, y_sc8, y_sc32)]
            with torch.cuda.device(x_fp8.device):
                out = torch.empty(tuple(x_fp8.shape), dtype=torch.float32, device=x_fp8.device)
                check(lib.pb_elementwise(code, xs[0].data_ptr(), _DTYPE_FMT[x_fp8.dtype], xs[1].data_ptr(), xs[2].data_ptr(),
                                         xs[3].data_ptr(), _DTYPE_FMT[y_fp8.dtype], xs[4].data_ptr(), xs[5].data_ptr(),
                                         math.prod(shape[:-2]), shape[-2], shape[-1], a, b, out.data_ptr(), _stream(x_fp8)))
            return out
        x = dequantize_impl(x_fp8, x_sc8, x_sc32, torch.float32, tgrid)
        y = dequantize_impl(y_fp8, y_sc8, y_sc32, torch.float32, tgrid)
        return op(x, y)
    return impl


add_impl = make_elementwise_impl(torch.add)
mul_impl = make_elementwise_impl(torch.mul)
sub_impl = make_elementwise_impl(torch.sub)
truediv_impl = make_elementwise_impl(torch.div)
floordiv_impl = make_elementwise_impl(torch.floor_divide)
mod_impl = make_elementwise_impl(torch.remainder)
pow_impl = make_elementwise_impl(torch.pow)


add_impl_bwd = make_elementwise_impl_bwd(torch.add)
mul_impl_bwd = make_elementwise_impl_bwd(torch.mul)
sub_impl_bwd = make_elementwise_impl_bwd(torch.sub)
truediv_impl_bwd = make_elementwise_impl_bwd(torch.div)
floordiv_impl_bwd = make_elementwise_impl_bwd(torch.floor_divide)
mod_impl_bwd = make_elementwise_impl_bwd(torch.remainder)
pow_impl_bwd = make_elementwise_impl_bwd(torch.pow)
