"""The WKV-7 state scan of the reference's TimeMix block (pratchya/_nnx_impl/_module.py:187-207) as one
CUDA kernel.  The projections, token shift, rotary embedding, normalisations and gates around the scan
(:129-186, :209-217) are the model's glue and stay with the caller."""
from __future__ import annotations

import torch

from .. import _lib
from .._lib import check


def wkv_state_scan(wkv_state, decay, iclr, removal_k, replacement_k, v, r, n_head: int):
    """(wkv_state', out): the scan of :187-207 over the T timesteps of six f32 [B, T, C] inputs from the
    initial state wkv_state [B, N, H, H] (None: zeros), with C = N * H and H = 64.  `out` is [B, T, C]
    (the reference's order after its transpose, :210)."""
    ins = [decay, iclr, removal_k, replacement_k, v, r]
    for t in ins:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError("wkv_state_scan inputs must be CUDA tensors: pratchya_b200 has no CPU path")
    shape = tuple(decay.shape)
    if len(shape) != 3 or any(tuple(t.shape) != shape for t in ins):
        raise ValueError("the six inputs must share one [B, T, C] shape")
    bsz, steps, chans = shape
    if chans % n_head:
        raise ValueError(f"{chans} channels do not split into {n_head} heads")
    head_dim = chans // n_head
    ins = [t.to(torch.float32).contiguous() for t in ins]            # the reference casts to f32 before the scan (:153-184)
    dev = decay.device
    lib = _lib.load()
    with torch.cuda.device(dev):
        state_in = None
        if wkv_state is not None:
            state_in = wkv_state.to(torch.float32).contiguous()
            if tuple(state_in.shape) != (bsz, n_head, head_dim, head_dim):
                raise ValueError(f"wkv_state has shape {tuple(state_in.shape)}, expected {(bsz, n_head, head_dim, head_dim)}")
        out = torch.empty(shape, dtype=torch.float32, device=dev)
        state_out = torch.empty((bsz, n_head, head_dim, head_dim), dtype=torch.float32, device=dev)
        check(lib.pb_wkv7_forward(*[t.data_ptr() for t in ins], state_in.data_ptr() if state_in is not None else None,
                                  bsz, steps, n_head, head_dim, out.data_ptr(), state_out.data_ptr(),
                                  torch.cuda.current_stream(dev).cuda_stream))
    return state_out, out
