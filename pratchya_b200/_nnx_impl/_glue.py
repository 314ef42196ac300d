"""Fused f32 glue of the modified RWKV-7 block (pratchya/_nnx_impl/_module.py:129-258) on the kernels of
csrc/rwkv_glue.cu: token shift + lerps, and everything between TimeMix's linears and its scan.  Each function is
differentiable (torch.autograd.Function around the forward and the backward kernel) and takes/returns f32 CUDA
tensors [B, T, C]."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .._lib import check


def _f32c(t):
    return t.to(torch.float32).contiguous()


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


class _ShiftLerpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, state, mu):
        lib = _lib.load()
        bsz, steps, chans = x.shape
        n_mix = mu.shape[0]
        out = torch.empty((n_mix, bsz, steps, chans), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.pb_token_shift_lerp(x.data_ptr(), state.data_ptr() if state is not None else None, mu.data_ptr(),
                                          bsz, steps, chans, n_mix, out.data_ptr(), _stream(x.device)))
        ctx.save_for_backward(x, state, mu)
        return tuple(out.unbind(0))          # separate outputs: their cotangents arrive separately, with no stacking copy

    @staticmethod
    def backward(ctx, *gs):
        x, state, mu = ctx.saved_tensors
        lib = _lib.load()
        bsz, steps, chans = x.shape
        n_mix = mu.shape[0]
        dev = x.device
        with torch.cuda.device(dev):
            gs = [_f32c(g) if g is not None else torch.zeros_like(x) for g in gs]
            g_ptrs = (C.c_void_p * n_mix)(*[g.data_ptr() for g in gs])
            dx = torch.empty_like(x)
            dstate = torch.empty_like(state) if state is not None else None
            dmu = torch.empty_like(mu)
            ws_bytes = lib.pb_token_shift_lerp_bwd_workspace_size(bsz, steps, chans, n_mix)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_token_shift_lerp_bwd(g_ptrs, x.data_ptr(), state.data_ptr() if state is not None else None, mu.data_ptr(),
                                              bsz, steps, chans, n_mix, dx.data_ptr(), dstate.data_ptr() if dstate is not None else None,
                                              dmu.data_ptr(), ws.data_ptr(), ws_bytes, _stream(dev)))
        return dx, dstate, dmu


def token_shift_lerp(x, state, mu):
    """[lerp(x, shifted(x), mu[k]) for k]: x [B, T, C], state [B, 1, C] (the token before the first; None: zeros),
    mu [n_mix, C] with n_mix 1 or 6.  Returns a tuple of n_mix tensors [B, T, C].  _module.py:137-151, :240-247."""
    if x.dim() != 3 or mu.dim() != 2 or mu.shape[1] != x.shape[2] or mu.shape[0] not in (1, 6):
        raise ValueError(f"token_shift_lerp: x {tuple(x.shape)}, mu {tuple(mu.shape)}")
    if not x.is_cuda:
        raise RuntimeError("token_shift_lerp needs CUDA tensors: pratchya_b200 has no CPU path")
    st = None
    if state is not None:
        if tuple(state.shape) != (x.shape[0], 1, x.shape[2]):
            raise ValueError(f"token_shift_lerp: state {tuple(state.shape)} for x {tuple(x.shape)}")
        st = _f32c(state)
    return _ShiftLerpFn.apply(_f32c(x), st, _f32c(mu))


class QuantizedMix:
    """One output of token_shift_lerp_quantized: everything a Linear needs of its input, without the input.
    `handle` is a [B, T, C] f32 tensor of stride zero (no memory behind it) that carries the autograd edge: a Linear
    takes it as its x, never reads it, and returns the cotangent of the mix for it.  `row` is the triple of
    quantize_impl(mix, (1,128)) over [B*T, C]; `tokens` the triple of quantize_impl(mix^T, (1,128)) or None."""
    __slots__ = ("handle", "row", "tokens")

    def __init__(self, handle, row, tokens):
        self.handle, self.row, self.tokens = handle, row, tokens

    @property
    def shape(self):
        return self.handle.shape


class _ShiftLerpQuantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, state, mu, mask):
        lib = _lib.load()
        bsz, steps, chans = x.shape
        n_mix, rows = mu.shape[0], bsz * steps
        n_t = bin(mask).count("1")
        dev = x.device
        groups = rows * chans // 1024
        with torch.cuda.device(dev):
            q = torch.empty((n_mix, rows, chans), dtype=torch.float8_e4m3fn, device=dev)
            sc8 = torch.empty((n_mix, groups, 8), dtype=torch.float8_e8m0fnu, device=dev)
            sc32 = torch.empty((n_mix, groups, 1, 1), dtype=torch.float32, device=dev)
            q_t = torch.empty((n_t, chans, rows), dtype=torch.float8_e4m3fn, device=dev)
            sc8_t = torch.empty((n_t, groups, 8), dtype=torch.float8_e8m0fnu, device=dev)
            sc32_t = torch.empty((n_t, groups, 1, 1), dtype=torch.float32, device=dev)
            check(lib.pb_shift_lerp_quantize(x.data_ptr(), state.data_ptr() if state is not None else None, mu.data_ptr(), bsz, steps, chans, n_mix,
                                             q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), mask,
                                             q_t.data_ptr() if n_t else None, sc8_t.data_ptr() if n_t else None, sc32_t.data_ptr() if n_t else None,
                                             _stream(dev)))
            handles = tuple(torch.zeros(1, dtype=torch.float32, device=dev).expand(bsz, steps, chans) for _ in range(n_mix))
        ctx.save_for_backward(x, state, mu)
        ctx.mark_non_differentiable(q, sc8, sc32, q_t, sc8_t, sc32_t)
        ctx.set_materialize_grads(False)      # no zero-filled fp8 arrays for the triples' absent cotangents
        return (*handles, q, sc8, sc32, q_t, sc8_t, sc32_t)

    @staticmethod
    def backward(ctx, *gs):
        n_mix = ctx.saved_tensors[2].shape[0]
        return (*_ShiftLerpFn.backward(ctx, *gs[:n_mix]), None)


def token_shift_lerp_quantized(x, state, mu, transposed=()):
    """token_shift_lerp whose mixes leave as fp8 triples for the Linears that consume them (a Linear quantizes its
    input on (1,128) first, _module.py:46-47): returns one QuantizedMix per row of mu.  `transposed`: the indices of
    the mixes that also get the triple of their transpose (the wgrad operand of a (128,128) Linear); it needs
    T % 1024 == 0.  C must be a multiple of 1024.  The bytes are those of token_shift_lerp + quantize_impl /
    quantize_transposed_impl; the mixes themselves are never written."""
    if x.dim() != 3 or mu.dim() != 2 or mu.shape[1] != x.shape[2] or mu.shape[0] not in (1, 6):
        raise ValueError(f"token_shift_lerp_quantized: x {tuple(x.shape)}, mu {tuple(mu.shape)}")
    if not x.is_cuda:
        raise RuntimeError("token_shift_lerp_quantized needs CUDA tensors: pratchya_b200 has no CPU path")
    st = None
    if state is not None:
        if tuple(state.shape) != (x.shape[0], 1, x.shape[2]):
            raise ValueError(f"token_shift_lerp_quantized: state {tuple(state.shape)} for x {tuple(x.shape)}")
        st = _f32c(state)
    n_mix = mu.shape[0]
    mask = 0
    for k in transposed:
        if not 0 <= k < n_mix:
            raise ValueError(f"token_shift_lerp_quantized: transposed index {k} of {n_mix} mixes")
        mask |= 1 << k
    out = _ShiftLerpQuantFn.apply(_f32c(x), st, _f32c(mu), mask)
    handles, (q, sc8, sc32, q_t, sc8_t, sc32_t) = out[:n_mix], out[n_mix:]
    mixes, slot = [], 0
    for k in range(n_mix):
        tokens = None
        if mask >> k & 1:
            tokens, slot = (q_t[slot], sc8_t[slot], sc32_t[slot]), slot + 1
        mixes.append(QuantizedMix(handles[k], (q[k], sc8[k], sc32[k]), tokens))
    return tuple(mixes)


def can_quantize_mixes(x, want_transposed):
    """Whether token_shift_lerp_quantized applies to x [B, T, C]."""
    return x.dim() == 3 and x.shape[2] % 1024 == 0 and x.numel() > 0 and (not want_transposed or x.shape[1] % 1024 == 0)


class _WkvPrepareFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt, n_head):
        lib = _lib.load()
        bsz, steps, chans = r_raw.shape
        outs = [torch.empty_like(r_raw) for _ in range(7)]
        with torch.cuda.device(r_raw.device):
            check(lib.pb_wkv_prepare(r_raw.data_ptr(), k_raw.data_ptr(), d.data_ptr(), iclr_raw.data_ptr(), v_prime.data_ptr(),
                                     v0.data_ptr() if v0 is not None else None, nu_raw.data_ptr() if nu_raw is not None else None,
                                     cos_tab.data_ptr(), sin_tab.data_ptr(), rk_mult.data_ptr(), mix_amt.data_ptr(),
                                     bsz, steps, n_head, chans // n_head, *[o.data_ptr() for o in outs], _stream(r_raw.device)))
        ctx.save_for_backward(r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt)
        ctx.n_head = n_head
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt = ctx.saved_tensors
        lib = _lib.load()
        bsz, steps, chans = r_raw.shape
        n_head = ctx.n_head
        dev = r_raw.device
        with torch.cuda.device(dev):
            gs = [_f32c(g) if g is not None else torch.zeros_like(r_raw) for g in grads]
            douts = [torch.empty_like(r_raw) for _ in range(5)]
            d_v0 = torch.empty_like(r_raw) if v0 is not None else None
            d_nu = torch.empty_like(r_raw) if v0 is not None else None
            d_rk, d_mix = torch.empty_like(rk_mult), torch.empty_like(mix_amt)
            ws_bytes = lib.pb_wkv_prepare_bwd_workspace_size(bsz, steps, n_head, chans // n_head)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_wkv_prepare_bwd(r_raw.data_ptr(), k_raw.data_ptr(), d.data_ptr(), iclr_raw.data_ptr(), v_prime.data_ptr(),
                                         v0.data_ptr() if v0 is not None else None, nu_raw.data_ptr() if nu_raw is not None else None,
                                         cos_tab.data_ptr(), sin_tab.data_ptr(), rk_mult.data_ptr(), mix_amt.data_ptr(),
                                         bsz, steps, n_head, chans // n_head, *[g.data_ptr() for g in gs],
                                         *[o.data_ptr() for o in douts], d_v0.data_ptr() if d_v0 is not None else None,
                                         d_nu.data_ptr() if d_nu is not None else None, d_rk.data_ptr(), d_mix.data_ptr(),
                                         ws.data_ptr(), ws_bytes, _stream(dev)))
        d_r_raw, d_k_raw, d_d, d_iclr_raw, d_v_prime = douts
        return d_r_raw, d_k_raw, d_d, d_iclr_raw, d_v_prime, d_v0, d_nu, None, None, d_rk, d_mix, None


def wkv_prepare(r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt, n_head: int):
    """(decay, iclr, removal_k, replacement_k, v, r, k) of TimeMix (_module.py:157-184) from the outputs of its
    linears: all [B, T, C] f32; v0 / nu_raw None in the first layer; cos_tab / sin_tab [T, 32]; rk_mult and mix_amt
    [C] (or [1, C]) as read through their quantization.  Head size 64."""
    ins = [r_raw, k_raw, d, iclr_raw, v_prime]
    shape = tuple(r_raw.shape)
    if len(shape) != 3 or any(tuple(t.shape) != shape for t in ins) or shape[2] != n_head * 64:
        raise ValueError(f"wkv_prepare: inputs must share a shape [B, T, {n_head} * 64], got {[tuple(t.shape) for t in ins]}")
    if (v0 is None) != (nu_raw is None):
        raise ValueError("wkv_prepare: v0 and nu_raw come together")
    if not r_raw.is_cuda:
        raise RuntimeError("wkv_prepare needs CUDA tensors: pratchya_b200 has no CPU path")
    if tuple(cos_tab.shape) != (shape[1], 32) or tuple(sin_tab.shape) != (shape[1], 32):
        raise ValueError(f"wkv_prepare: angle tables must be [{shape[1]}, 32]")
    ins = [_f32c(t) for t in ins]
    opt = [_f32c(t) if t is not None else None for t in (v0, nu_raw)]
    return _WkvPrepareFn.apply(*ins, *opt, _f32c(cos_tab), _f32c(sin_tab), _f32c(rk_mult).reshape(-1), _f32c(mix_amt).reshape(-1), n_head)


class _RmsNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps):
        lib = _lib.load()
        chans = x.shape[-1]
        rows = x.numel() // chans
        y = torch.empty_like(x)
        inv = torch.empty(rows, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.pb_rms_norm(x.data_ptr(), scale.data_ptr(), rows, chans, eps, y.data_ptr(), inv.data_ptr(), _stream(x.device)))
        ctx.save_for_backward(x, scale, inv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, scale, inv = ctx.saved_tensors
        lib = _lib.load()
        chans = x.shape[-1]
        rows = x.numel() // chans
        dy = _f32c(dy)
        dev = x.device
        with torch.cuda.device(dev):
            dx, dscale = torch.empty_like(x), torch.empty_like(scale)
            ws_bytes = lib.pb_rms_norm_bwd_workspace_size(rows, chans)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_rms_norm_bwd(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), inv.data_ptr(), rows, chans,
                                      dx.data_ptr(), dscale.data_ptr(), ws.data_ptr(), ws_bytes, _stream(dev)))
        return dx, dscale, None


def rms_norm(x, scale, eps: float):
    """(x * rsqrt(mean(x^2, -1) + eps)) * scale, _module.py:61-72; x [..., C] f32, scale [C] or [1, C] as read through its
    quantization; C a multiple of 128."""
    if not x.is_cuda:
        raise RuntimeError("rms_norm needs CUDA tensors: pratchya_b200 has no CPU path")
    if scale.numel() != x.shape[-1] or x.shape[-1] % 128 != 0:
        raise ValueError(f"rms_norm: x {tuple(x.shape)}, scale {tuple(scale.shape)} (the last dimension must be a multiple of 128)")
    return _RmsNormFn.apply(_f32c(x), _f32c(scale).reshape(-1), float(eps))


class _Relu2Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        lib = _lib.load()
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            check(lib.pb_relu2(x.data_ptr(), x.numel(), y.data_ptr(), _stream(x.device)))
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, g):
        (x,) = ctx.saved_tensors
        lib = _lib.load()
        g = _f32c(g)
        dx = torch.empty_like(x)
        with torch.cuda.device(x.device):
            check(lib.pb_relu2_bwd(g.data_ptr(), x.data_ptr(), x.numel(), dx.data_ptr(), _stream(x.device)))
        return dx


def relu2(x):
    """relu(x) ** 2, _module.py:249; the element count must be a multiple of 4."""
    if not x.is_cuda:
        raise RuntimeError("relu2 needs CUDA tensors: pratchya_b200 has no CPU path")
    return _Relu2Fn.apply(_f32c(x))


class _Relu2QuantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k):
        lib = _lib.load()
        cols = k.shape[-1]
        rows = k.numel() // cols
        groups = rows * cols // 1024
        dev = k.device
        with torch.cuda.device(dev):
            q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=dev)
            sc8 = torch.empty((groups, 8), dtype=torch.float8_e8m0fnu, device=dev)
            sc32 = torch.empty((groups, 1, 1), dtype=torch.float32, device=dev)
            q_t = torch.empty((cols, rows), dtype=torch.float8_e4m3fn, device=dev)
            sc8_t = torch.empty((groups, 8), dtype=torch.float8_e8m0fnu, device=dev)
            sc32_t = torch.empty((groups, 1, 1), dtype=torch.float32, device=dev)
            check(lib.pb_relu2_quantize_dual(k.data_ptr(), rows, cols, q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                                             q_t.data_ptr(), sc8_t.data_ptr(), sc32_t.data_ptr(), _stream(dev)))
            handle = torch.zeros(1, dtype=torch.float32, device=dev).expand(k.shape)
        ctx.save_for_backward(k)
        ctx.mark_non_differentiable(q, sc8, sc32, q_t, sc8_t, sc32_t)
        ctx.set_materialize_grads(False)
        return handle, q, sc8, sc32, q_t, sc8_t, sc32_t

    @staticmethod
    def backward(ctx, g, *_):
        if g is None:
            return None
        return _Relu2Fn.backward(ctx, g)


def relu2_quantized(k):
    """relu(k) ** 2 (_module.py:249) for a consumer that is a (128,128) Linear with a backward pass to follow: the result
    leaves as a QuantizedMix (the (1,128) triple and the triple of the transpose) and is never written as f32.  k [..., C] f32
    with C and the number of rows multiples of 1024.  The bytes are those of relu2 + quantize_impl / quantize_transposed_impl."""
    if not k.is_cuda:
        raise RuntimeError("relu2_quantized needs CUDA tensors: pratchya_b200 has no CPU path")
    out = _Relu2QuantFn.apply(_f32c(k))
    return QuantizedMix(out[0], (out[1], out[2], out[3]), (out[4], out[5], out[6]))


def can_quantize_relu2(k):
    return k.is_cuda and k.dim() >= 2 and k.shape[-1] % 1024 == 0 and k.numel() > 0 and (k.numel() // k.shape[-1]) % 1024 == 0


class _WkvFinishFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, eps, n_head):
        lib = _lib.load()
        bsz, steps, chans = y.shape
        dev = y.device
        out = torch.empty_like(y)
        stats = torch.empty((bsz * n_head, 2), dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            ws_bytes = lib.pb_wkv_finish_workspace_size(bsz, steps, n_head, chans // n_head)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_wkv_finish(y.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), gate.data_ptr(), gn_scale.data_ptr(),
                                    gn_bias.data_ptr(), bonus_mult.data_ptr(), eps, bsz, steps, n_head, chans // n_head,
                                    out.data_ptr(), stats.data_ptr(), ws.data_ptr(), ws_bytes, _stream(dev)))
        ctx.save_for_backward(y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, stats)
        ctx.n_head = n_head
        return out

    @staticmethod
    def backward(ctx, g):
        y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, stats = ctx.saved_tensors
        lib = _lib.load()
        bsz, steps, chans = y.shape
        n_head = ctx.n_head
        dev = y.device
        g = _f32c(g)
        with torch.cuda.device(dev):
            d_y, d_r, d_k, d_v, d_gate = (torch.empty_like(y) for _ in range(5))
            d_gs, d_gb, d_bm = torch.empty_like(gn_scale), torch.empty_like(gn_bias), torch.empty_like(bonus_mult)
            ws_bytes = lib.pb_wkv_finish_bwd_workspace_size(bsz, steps, n_head, chans // n_head)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_wkv_finish_bwd(g.data_ptr(), y.data_ptr(), r.data_ptr(), k.data_ptr(), v.data_ptr(), gate.data_ptr(),
                                        gn_scale.data_ptr(), gn_bias.data_ptr(), bonus_mult.data_ptr(), stats.data_ptr(),
                                        bsz, steps, n_head, chans // n_head, d_y.data_ptr(), d_r.data_ptr(), d_k.data_ptr(),
                                        d_v.data_ptr(), d_gate.data_ptr(), d_gs.data_ptr(), d_gb.data_ptr(), d_bm.data_ptr(),
                                        ws.data_ptr(), ws_bytes, _stream(dev)))
        return d_y, d_r, d_k, d_v, d_gate, d_gs, d_gb, d_bm, None, None


def wkv_finish(y, r, k, v, gate, gn_scale, gn_bias, bonus_mult, eps: float, n_head: int):
    """(GroupNorm(y) + sum_c(r * k * bonus_mult) * v) * gate of TimeMix (_module.py:208-216): y the scan's output, all
    [B, T, C] f32 with C = n_head * 64; gn_scale, gn_bias, bonus_mult [C] (or [1, C]); one norm group per head with
    statistics over the T x 64 values of a batch element (flax GroupNorm on [B, T, C], :118-123)."""
    ins = [y, r, k, v, gate]
    shape = tuple(y.shape)
    if len(shape) != 3 or any(tuple(t.shape) != shape for t in ins) or shape[2] != n_head * 64:
        raise ValueError(f"wkv_finish: inputs must share a shape [B, T, {n_head} * 64], got {[tuple(t.shape) for t in ins]}")
    if not y.is_cuda:
        raise RuntimeError("wkv_finish needs CUDA tensors: pratchya_b200 has no CPU path")
    return _WkvFinishFn.apply(*[_f32c(t) for t in ins], _f32c(gn_scale).reshape(-1), _f32c(gn_bias).reshape(-1),
                              _f32c(bonus_mult).reshape(-1), float(eps), n_head)


class _SmoothedXentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, weight, alpha, denominator, reuse_logits=False):
        lib = _lib.load()
        rows, vocab = logits.shape
        dev = logits.device
        row_loss = torch.empty(rows, dtype=torch.float32, device=dev)
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            check(lib.pb_smoothed_xent(logits.data_ptr(), target.data_ptr(), weight.data_ptr(), rows, vocab, alpha,
                                       row_loss.data_ptr(), lse.data_ptr(), _stream(dev)))
        ctx.save_for_backward(logits, target, weight, lse)
        ctx.alpha, ctx.denominator, ctx.reuse_logits = alpha, denominator, bool(reuse_logits)
        return row_loss.sum() / denominator

    @staticmethod
    def backward(ctx, g):
        logits, target, weight, lse = ctx.saved_tensors
        lib = _lib.load()
        rows, vocab = logits.shape
        dev = logits.device
        g = g.to(torch.float32).reshape(1).contiguous()
        # every element of the cotangent depends on its own logit only: with reuse_logits it is written over the logits
        dlogits = logits if ctx.reuse_logits else torch.empty_like(logits)
        with torch.cuda.device(dev):
            check(lib.pb_smoothed_xent_bwd(logits.data_ptr(), target.data_ptr(), weight.data_ptr(), lse.data_ptr(), g.data_ptr(),
                                           ctx.denominator, rows, vocab, ctx.alpha, dlogits.data_ptr(), _stream(dev)))
        return dlogits, None, None, None, None, None


def smoothed_cross_entropy(logits, labels, alpha: float = 0.1, reuse_logits: bool = False):
    """compute_loss, pratchya/_nnx_impl/_utils.py:7-13, on logits [B, T, V] f32 and labels [B, T]: position t predicts label
    t+1 (the reference's caller passes logits[:, :-1] and label[:, 1:]), one-hot labels smoothed by alpha, softmax cross
    entropy, mean over the B * (T-1) positions.  One pass over the logits forward and one backward.  `reuse_logits`: the
    backward pass writes the logits' cotangent over the logits themselves (8.6 GB less at the peak of a step with 32768
    tokens and 65536 words); for a caller that does not read the logits afterwards and runs the backward pass once."""
    if not logits.is_cuda:
        raise RuntimeError("smoothed_cross_entropy needs CUDA tensors: pratchya_b200 has no CPU path")
    bsz, steps, vocab = logits.shape
    if steps < 2 or tuple(labels.shape) != (bsz, steps) or vocab % 4 != 0:
        raise ValueError(f"smoothed_cross_entropy: logits {tuple(logits.shape)}, labels {tuple(labels.shape)}")
    target = torch.cat([labels[:, 1:], labels[:, :1]], dim=1).to(torch.int64).reshape(-1).contiguous()      # the last column is a placeholder
    weight = torch.ones(bsz, steps, dtype=torch.float32, device=logits.device)
    weight[:, -1] = 0.0
    flat = _f32c(logits).reshape(bsz * steps, vocab)
    reuse = bool(reuse_logits) and flat.data_ptr() == logits.data_ptr()          # only the caller's own array, never a converted copy's alias
    return _SmoothedXentFn.apply(flat, target, weight.reshape(-1), float(alpha), float(bsz * (steps - 1)), reuse)
