"""world_size-2 gloo run of the end-to-end step's only collective: pratchya_b200._nnx_impl._dp.allreduce_gradients."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pratchya_b200._nnx_impl._dp import allreduce_gradients
        shapes = [(3, 5), (7,), (2, 2, 2)]
        params = [torch.nn.Parameter(torch.zeros(s)) for s in shapes]
        full = []
        for r in range(world):                                   # every rank can form every rank's gradients: seeded
            gen = torch.Generator().manual_seed(10 + r)
            full.append([torch.randn(s, generator=gen) for s in shapes])
        for p, g in zip(params, full[rank]):
            p.grad = g.clone()
        if rank == 1:
            params[1].grad = None                                # a parameter one rank did not touch counts as zeros there
        full[1][1] = torch.zeros(shapes[1])
        sent = allreduce_gradients(params, world, wire_dtype=torch.bfloat16)
        want = [sum(f[i].to(torch.bfloat16) for f in full).to(torch.float32) / world for i in range(len(shapes))]
        ok = sent == sum(p.numel() for p in params) * 2
        for p, w in zip(params, want):
            ok = ok and p.grad is not None and torch.allclose(p.grad, w, rtol=2e-2, atol=2e-2)    # bf16 on the wire
        gathered = [None] * world
        dist.all_gather_object(gathered, [p.grad.clone() for p in params])
        same = all(torch.equal(a, b) for a, b in zip(gathered[0], gathered[1]))                   # both ranks hold the same average
        if rank == 0:
            ret["ok"] = bool(ok and same)
    finally:
        dist.destroy_process_group()


def test_two_ranks_average_their_gradients():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert ret.get("ok") is True


def test_single_rank_is_a_no_op():
    from pratchya_b200._nnx_impl._dp import allreduce_gradients
    p = torch.nn.Parameter(torch.ones(4))
    p.grad = torch.full((4,), 3.0)
    assert allreduce_gradients([p], 1) == 0 and torch.equal(p.grad, torch.full((4,), 3.0))


def _health_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pratchya_b200._nnx_impl._dp import FAILED, HEALTHY, OUT_OF_MEMORY, agree_on_health, run_guarded
        host_group = dist.new_group(backend="gloo")
        seen = []

        def work(step):
            def fn():
                if step == 1 and rank == 1:
                    raise RuntimeError("unspecified launch failure (injected on the host)")
                if step == 2 and rank == 0:
                    raise torch.OutOfMemoryError("injected")
            return fn

        for step in range(3):
            code, msg = run_guarded(work(step), sync=lambda: None)
            worst = agree_on_health(code, world, host_group)
            seen.append((code, worst, msg))
            # a healthy step would now enter the collective; an unhealthy one is left by every rank at this same point
            if worst == HEALTHY:
                t = torch.ones(1)
                dist.all_reduce(t)
                assert t.item() == world
        want_codes = {0: [HEALTHY, HEALTHY, OUT_OF_MEMORY], 1: [HEALTHY, FAILED, HEALTHY]}[rank]
        ok = [c for c, _, _ in seen] == want_codes and [w for _, w, _ in seen] == [HEALTHY, FAILED, OUT_OF_MEMORY]
        ok = ok and (seen[1][2] is None) == (rank == 0)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_ranks_agree_that_one_of_them_failed_before_the_collective():
    """The step before the gradient exchange: a rank whose work raised (a kernel fault, an allocation failure: injected
    on the host here) reports it through the host group, every rank sees the worst code and none enters the
    collective of that step."""
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_health_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert ret.get(0) is True and ret.get(1) is True
