"""Row (token) sharding of the quantize / GEMM path across the GPUs of one box.

No exchange step exists on this path: (1, b) block scaling is local to a row, and a
super-group is 8 consecutive blocks in row-major order, so a shard reproduces the bytes of
the unsharded run whenever its boundaries fall on super-group boundaries.
"""
from __future__ import annotations

import math


def shard_alignment(cols: int, b: int = 128, transposed_b: int | None = None) -> int:
    """Smallest row multiple at which a [rows, cols] activation may be cut so that every shard
    quantizes to the same bytes as the full tensor on grid (1, b): the shard must start on a
    super-group boundary, i.e. hold a multiple of 8 blocks before it (pratchya/_qualia/_qarr.py:474-485).
    `transposed_b` adds the wgrad operand's constraint (token blocks of `transposed_b` rows,
    8 per super-group)."""
    nbc = cols // b
    k = max(1, b // 16)
    align = k // math.gcd(k, nbc)
    if transposed_b:
        align = math.lcm(align, transposed_b * max(1, transposed_b // 16))
    return align


def row_shard(rows: int, world: int, rank: int, align: int = 1):
    """[start, stop) of rank's rows: `rows` split as evenly as `align` allows."""
    if rows % align:
        raise ValueError(f"rows={rows} is not a multiple of the shard alignment {align}")
    units = rows // align
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * align, stop * align
