"""A second, independently written restatement of the reference's quantize / dequantize rule, on torch CPU
tensors, compared with the numpy oracle on the committed golden inputs and on larger seeded ones.

It follows the reference's text (pratchya/_qualia/_qarr.py:470-506 and :550-569) with a different
toolkit -- torch's casts and reductions instead of numpy + ml_dtypes, a gather of blocks by index
arithmetic instead of a reshape/transpose chain -- so a misreading of the rule would have to be made
twice, in two idioms, to go unnoticed.  It cannot pin the oracle to the reference's own output (none
exists here: the reference has no tests or vectors and cannot be imported), only to a second reading."""
import math
from pathlib import Path

import ml_dtypes
import numpy as np
import pytest
import torch

from oracle import qarr_oracle as o

GOLDEN = np.load(Path(__file__).parent / "golden" / "quant_golden.npz")
NAMES = sorted({k.split(".")[0] for k in GOLDEN.files})


def _block_index(rows, cols, a, b):
    """For every element of a [rows, cols] array the number of its (a, b) block, blocks counted along the
    block grid's rows first (the order the reference's transpose puts them in, :470-472)."""
    r = torch.arange(rows).unsqueeze(1) // a
    c = torch.arange(cols).unsqueeze(0) // b
    return r * (cols // b) + c


def second_quantize(x: torch.Tensor, tgrid):
    a, b = tgrid
    rows, cols = x.shape
    nblocks = (rows // a) * (cols // b)
    k = math.gcd(max(1, (a * b) // 16), nblocks)                       # :477-478
    m = nblocks // k                                                   # :480
    blk = _block_index(rows, cols, a, b).reshape(-1)
    absx = x.abs().reshape(-1).to(torch.float32)
    m_i = torch.zeros(nblocks, dtype=torch.float32).scatter_reduce(0, blk, absx, reduce="amax", include_self=True)    # :484
    big = m_i.reshape(m, k).amax(dim=1)                                # :485
    safe = torch.where(big == 0, torch.ones_like(big), big)            # :488
    s = m_i.reshape(m, k) / safe.unsqueeze(1)                          # :489
    sb = (s.contiguous().view(torch.int32) >> 23).to(torch.uint8)      # :492-493
    s_q = (sb.to(torch.int32) << 23).view(torch.float32)               # :495
    s_eff = torch.maximum(s_q * big.unsqueeze(1), torch.tensor(1e-7, dtype=torch.float32))     # :496-497
    per_elem = s_eff.reshape(-1)[blk].reshape(rows, cols)
    v = x.to(torch.float32) / per_elem * 128.0                         # :499
    q = v.to(torch.bfloat16).to(torch.float8_e4m3fn)
    return q, sb, big.reshape(m, 1, 1)


def second_dequantize(q, sb, big, tgrid, dtype):
    a, b = tgrid
    rows, cols = q.shape
    m, k = sb.shape                                                    # :550
    blk = _block_index(rows, cols, a, b).reshape(-1)
    x_sc = (sb.to(torch.int32) << 23).view(torch.float32) * big.reshape(m, 1)     # :562-563
    per_elem = x_sc.reshape(-1)[blk].reshape(rows, cols)
    return (q.to(torch.bfloat16).to(torch.float32) * per_elem / 128.0).to(dtype)  # :564, :569


def _compare(x, grid):
    q, s8, s32 = o.quantize_impl(x, grid)
    tq, t8, t32 = second_quantize(torch.from_numpy(x), grid)
    assert np.array_equal(tq.view(torch.uint8).numpy(), q.view(np.uint8)), "fp8 bytes differ between the two restatements"
    assert np.array_equal(t8.numpy(), s8) and np.array_equal(t32.numpy().view(np.uint32), s32.view(np.uint32))
    for np_dt, t_dt in ((np.float32, torch.float32), (ml_dtypes.bfloat16, torch.bfloat16)):
        dq = o.dequantize_impl(q, s8, s32, np_dt, grid)
        tdq = second_dequantize(tq, t8, t32, grid, t_dt)
        if t_dt == torch.bfloat16:
            assert np.array_equal(tdq.view(torch.uint16).numpy(), dq.view(np.uint16))
        else:
            assert np.array_equal(tdq.numpy().view(np.uint32), dq.view(np.uint32))


@pytest.mark.parametrize("name", NAMES)
def test_second_restatement_agrees_with_the_oracle_on_the_golden_inputs(name):
    x, grid = GOLDEN[f"{name}.x"], tuple(int(v) for v in GOLDEN[f"{name}.grid"])
    _compare(x, grid)
    # and both agree with the committed bytes
    tq, t8, t32 = second_quantize(torch.from_numpy(x), grid)
    assert np.array_equal(tq.view(torch.uint8).numpy(), GOLDEN[f"{name}.q"])
    assert np.array_equal(t8.numpy(), GOLDEN[f"{name}.sc8"]) and np.array_equal(t32.numpy(), GOLDEN[f"{name}.sc32"])


@pytest.mark.parametrize("shape,grid,kind", [((512, 2048), (1, 128), "outliers"), ((512, 1024), (128, 128), "weights"),
                                             ((256, 64), (128, 1), "weights"), ((64, 96), (16, 16), "student_t"),
                                             ((48, 48), (1, 1), "outliers"), ((2048, 2048), (1, 128), "config1")])
def test_second_restatement_agrees_with_the_oracle_on_seeded_inputs(shape, grid, kind):
    rng = np.random.default_rng(hash((shape, grid)) % (1 << 31))
    if kind == "student_t":
        x = rng.standard_t(3, size=shape).astype(np.float32)
    elif kind == "weights":
        x = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    else:
        x = rng.standard_normal(shape).astype(np.float32)
        x[rng.random(shape) < 0.01] *= 64
    if kind == "config1":                      # BASELINE configs[0]: a bf16 tensor
        x = x.astype(ml_dtypes.bfloat16).astype(np.float32)
    x.reshape(-1)[:7] = 0.0                    # a few exact zeros
    _compare(x, grid)


def test_second_restatement_on_the_rule_s_corner_cases():
    x = np.zeros((4, 1024), dtype=np.float32)
    x[1, :128] = 3.0                   # one constant block alone in its super-group
    x[2, 5] = 1e-9                     # a super-group below the 1e-7 floor
    x[3, 0], x[3, 200] = 1.0, -2.0 ** -9
    _compare(x, (1, 128))
    _compare(np.full((128, 128), -0.0, dtype=np.float32), (128, 128))
