"""The WKV-7 state scan of the reference's TimeMix block (pratchya/_nnx_impl/_module.py:187-207) as CUDA
kernels: the scan itself and its cotangents (what jax.grad derives from the reference's nnx.scan), tied
together as a torch.autograd.Function.  The projections, token shift, rotary embedding, normalisations
and gates around the scan (:129-186, :209-217) are the model's glue and stay with the caller."""
from __future__ import annotations

import torch

from .. import _lib
from .._lib import check


def _check_inputs(ins, n_head):
    for t in ins:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError("wkv_state_scan inputs must be CUDA tensors: pratchya_b200 has no CPU path")
    shape = tuple(ins[0].shape)
    if len(shape) != 3 or any(tuple(t.shape) != shape for t in ins):
        raise ValueError("the six inputs must share one [B, T, C] shape")
    if shape[2] % n_head:
        raise ValueError(f"{shape[2]} channels do not split into {n_head} heads")
    return shape


def _forward(state_in, ins, n_head, want_checkpoints):
    bsz, steps, chans = ins[0].shape
    head_dim = chans // n_head
    dev = ins[0].device
    lib = _lib.load()
    with torch.cuda.device(dev):
        out = torch.empty((bsz, steps, chans), dtype=torch.float32, device=dev)
        state_out = torch.empty((bsz, n_head, head_dim, head_dim), dtype=torch.float32, device=dev)
        ckpt = sa = None
        if want_checkpoints:
            n_floats = lib.pb_wkv7_checkpoint_floats(bsz, steps, n_head, head_dim)
            if n_floats == 0:
                raise _lib.PbError(_lib.PB_ERR_UNSUPPORTED, f"wkv_state_scan: head size {head_dim} is not supported")
            ckpt = torch.empty(n_floats, dtype=torch.float32, device=dev)
            sa = torch.empty((bsz, steps, chans), dtype=torch.float32, device=dev)
        check(lib.pb_wkv7_forward(*[t.data_ptr() for t in ins], state_in.data_ptr() if state_in is not None else None,
                                  bsz, steps, n_head, head_dim, out.data_ptr(), state_out.data_ptr(),
                                  ckpt.data_ptr() if ckpt is not None else None, sa.data_ptr() if sa is not None else None,
                                  torch.cuda.current_stream(dev).cuda_stream))
    return state_out, out, ckpt, sa


class _WkvScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, state_in, decay, iclr, removal_k, replacement_k, v, r, n_head):
        ins = [t.contiguous() for t in (decay, iclr, removal_k, replacement_k, v, r)]
        state_out, out, ckpt, sa = _forward(state_in, ins, n_head, True)
        ctx.save_for_backward(*ins, ckpt, sa)
        ctx.n_head, ctx.has_state = n_head, state_in is not None
        return state_out, out

    @staticmethod
    def backward(ctx, d_state_out, d_out):
        *ins, ckpt, sa = ctx.saved_tensors
        bsz, steps, chans = ins[0].shape
        n_head = ctx.n_head
        head_dim = chans // n_head
        dev = ins[0].device
        lib = _lib.load()
        with torch.cuda.device(dev):
            d_out = d_out.to(torch.float32).contiguous() if d_out is not None else torch.zeros_like(ins[0])
            d_state = d_state_out.to(torch.float32).contiguous() if d_state_out is not None else None
            grads = [torch.empty_like(ins[0]) for _ in range(6)]
            d_state_in = torch.empty((bsz, n_head, head_dim, head_dim), dtype=torch.float32, device=dev) if ctx.has_state else None
            check(lib.pb_wkv7_backward(*[t.data_ptr() for t in ins], ckpt.data_ptr(), sa.data_ptr(), d_out.data_ptr(),
                                       d_state.data_ptr() if d_state is not None else None,
                                       bsz, steps, n_head, head_dim, *[g.data_ptr() for g in grads],
                                       d_state_in.data_ptr() if d_state_in is not None else None,
                                       torch.cuda.current_stream(dev).cuda_stream))
        return (d_state_in, *grads, None)


def wkv_state_scan(wkv_state, decay, iclr, removal_k, replacement_k, v, r, n_head: int):
    """(wkv_state', out): the scan of :187-207 over the T timesteps of six f32 [B, T, C] inputs from the
    initial state wkv_state [B, N, H, H] (None: zeros), with C = N * H and H = 64.  `out` is [B, T, C]
    (the reference's order after its transpose, :210).  Differentiable in the six inputs and the state."""
    ins = [decay, iclr, removal_k, replacement_k, v, r]
    shape = _check_inputs(ins, n_head)
    bsz, steps, chans = shape
    head_dim = chans // n_head
    ins = [t.to(torch.float32).contiguous() for t in ins]            # the reference casts to f32 before the scan (:153-184)
    state_in = None
    if wkv_state is not None:
        state_in = wkv_state.to(torch.float32).contiguous()
        if tuple(state_in.shape) != (bsz, n_head, head_dim, head_dim):
            raise ValueError(f"wkv_state has shape {tuple(state_in.shape)}, expected {(bsz, n_head, head_dim, head_dim)}")
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in ins + ([state_in] if state_in is not None else []))
    if needs_grad:
        return _WkvScanFn.apply(state_in, *ins, n_head)
    state_out, out, _, _ = _forward(state_in, ins, n_head, False)
    return state_out, out
