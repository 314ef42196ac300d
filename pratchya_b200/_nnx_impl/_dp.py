"""Data-parallel gradient exchange of the end-to-end step: the one collective of the training path.

Every rank runs the same model on its own sequences; after the backward pass the gradients are averaged with one
all-reduce of a flat bf16 buffer (the precision the benchmark configuration names for the exchange) and written
back into the parameters' .grad in f32.  torch.distributed does the transport (NCCL over NVLink on GPUs, gloo in
the CPU test); nothing here depends on the device.

`agree_on_health` is the step that comes before that collective: every rank finishes its own work of the step, and the
ranks then agree through a host-side group (CPU tensors, gloo) that all of them are healthy.  A rank whose work failed
says so there, so that no rank enters a device collective that another rank can no longer take part in."""
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


HEALTHY, OUT_OF_MEMORY, FAILED = 0, 1, 2


def run_guarded(fn, sync=None):
    """Runs fn() and then sync() (the device synchronize of the caller: a kernel fault of this rank surfaces there).
    Returns (code, message): HEALTHY, OUT_OF_MEMORY or FAILED with the exception's text."""
    try:
        fn()
        if sync is not None:
            sync()
        return HEALTHY, None
    except torch.OutOfMemoryError as e:
        return OUT_OF_MEMORY, f"OutOfMemoryError: {e}"[:300]
    except Exception as e:      # noqa: BLE001 - the text goes into the caller's record
        return FAILED, f"{type(e).__name__}: {e}"[:300]


def agree_on_health(code: int, world: int, host_group=None) -> int:
    """The worst of the ranks' codes, exchanged over CPU tensors only (`host_group`: a gloo group of all ranks; with one
    rank the code itself).  Every rank must call it at the same point of every step."""
    if world <= 1:
        return code
    t = torch.tensor([int(code)], dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=host_group)
    return int(t.item())
