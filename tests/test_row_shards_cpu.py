"""world_size-2 gloo run of the row-sharding logic: each rank quantizes its shard with the
oracle; the gathered shards must equal the unsharded result byte for byte (no collective is
needed on the data path, only this gather for the check)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pratchya_b200._shard import row_shard, shard_alignment


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, cols, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import qarr_oracle as o
        rng = np.random.default_rng(0)                     # same full tensor on every rank
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        x[rng.random((rows, cols)) < 0.01] *= 64
        lo, hi = row_shard(rows, world, rank, shard_alignment(cols))
        q, s8, s32 = o.quantize_impl(x[lo:hi], (1, 128))
        parts = [None] * world
        dist.all_gather_object(parts, (lo, hi, q.view(np.uint8), s8, s32))
        if rank == 0:
            fq, f8, f32 = o.quantize_impl(x, (1, 128))
            parts.sort(key=lambda p: p[0])
            assert parts[0][0] == 0 and parts[-1][1] == rows
            ok = (np.array_equal(np.concatenate([p[2] for p in parts]), fq.view(np.uint8))
                  and np.array_equal(np.concatenate([p[3] for p in parts]), f8)
                  and np.array_equal(np.concatenate([p[4] for p in parts]), f32))
            ret["ok"] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows,cols", [(64, 2048), (40, 512)])
def test_two_rank_row_shards_reproduce_the_full_tensor(rows, cols):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, rows, cols, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        assert ret.get("ok") is True


def test_shard_alignment_and_partition():
    assert shard_alignment(2048) == 1            # 16 blocks per row: every row starts a super-group
    assert shard_alignment(512) == 2             # 4 blocks per row: two rows per super-group
    assert shard_alignment(128) == 8
    assert shard_alignment(2048, transposed_b=128) == 1024
    assert row_shard(65536, 8, 3, 1024) == (24576, 32768)
    spans = [row_shard(10, 4, r) for r in range(4)]
    assert spans == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        row_shard(100, 2, 0, 8)
