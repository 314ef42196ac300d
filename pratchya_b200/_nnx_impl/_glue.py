"""Fused f32 glue of the modified RWKV-7 block (pratchya/_nnx_impl/_module.py:129-258) on the kernels of
csrc/rwkv_glue.cu: token shift + lerps, and everything between TimeMix's linears and its scan.  Each function is
differentiable (torch.autograd.Function around the forward and the backward kernel) and takes/returns f32 CUDA
tensors [B, T, C]."""
from __future__ import annotations

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
        return out

    @staticmethod
    def backward(ctx, g):
        x, state, mu = ctx.saved_tensors
        lib = _lib.load()
        bsz, steps, chans = x.shape
        n_mix = mu.shape[0]
        g = _f32c(g)
        dev = x.device
        with torch.cuda.device(dev):
            dx = torch.empty_like(x)
            dstate = torch.empty_like(state) if state is not None else None
            dmu = torch.empty_like(mu)
            ws_bytes = lib.pb_token_shift_lerp_bwd_workspace_size(bsz, steps, chans, n_mix)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            check(lib.pb_token_shift_lerp_bwd(g.data_ptr(), x.data_ptr(), state.data_ptr() if state is not None else None, mu.data_ptr(),
                                              bsz, steps, chans, n_mix, dx.data_ptr(), dstate.data_ptr() if dstate is not None else None,
                                              dmu.data_ptr(), ws.data_ptr(), ws_bytes, _stream(dev)))
        return dx, dstate, dmu


def token_shift_lerp(x, state, mu):
    """[lerp(x, shifted(x), mu[k]) for k]: x [B, T, C], state [B, 1, C] (the token before the first; None: zeros),
    mu [n_mix, C] with n_mix 1 or 6.  Returns [n_mix, B, T, C].  _module.py:137-151, :240-247."""
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
