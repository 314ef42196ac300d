"""Data-parallel gradient exchange of the end-to-end step: the one collective of the training path.

Every rank runs the same model on its own sequences; after the backward pass the gradients are averaged with one
all-reduce of a flat bf16 buffer (the precision the benchmark configuration names for the exchange) and written
back into the parameters' .grad in f32.  torch.distributed does the transport (NCCL over NVLink on GPUs, gloo in
the CPU test); nothing here depends on the device."""
from __future__ import annotations

import torch
import torch.distributed as dist


def allreduce_gradients(params, world: int, wire_dtype=torch.bfloat16) -> int:
    """Averages p.grad of every parameter over the `world` ranks of the default process group, in place.  Parameters
    without a gradient count as zeros.  Returns the number of bytes each rank put on the wire."""
    params = list(params)
    if world <= 1 or not params:
        return 0
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in params]).to(wire_dtype)
    dist.all_reduce(flat)
    avg = flat.to(torch.float32) / world
    off = 0
    for p in params:
        n = p.numel()
        g = avg[off:off + n].view_as(p).to(p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n
    return flat.numel() * flat.element_size()
