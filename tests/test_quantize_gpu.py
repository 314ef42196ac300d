"""GPU parity of the quantizer / dequantizer with the CPU oracle: fp8 bytes, e8m0 bytes
and fp32 scales must be bit-exact; dequantized values bit-exact too."""
import numpy as np
import pytest
import torch

from helpers import BF16, assert_triple_equal, bytes_of, from_torch, oracle, synth, to_torch
from pratchya_b200 import _lib
from pratchya_b200._qualia import dequantize_impl, dequantize_impl_bwd, quantize_impl

pytestmark = pytest.mark.gpu

GRIDS = [
    ((64, 2048), (1, 128)), ((2048, 2048), (1, 128)), ((8, 512), (1, 128)), ((3, 384), (1, 128)),
    ((256, 384), (128, 128)), ((1024, 1024), (128, 128)), ((2304, 1152), (128, 128)),
    ((256, 64), (128, 1)), ((64, 256), (1, 16)), ((64, 64), (16, 16)), ((8, 8), (1, 1)), ((32, 64), (4, 4)),
    ((12, 48), (3, 16)), ((64, 2048), (1, 32)), ((6, 10), (2, 5)),
]


@pytest.mark.parametrize("shape,grid", GRIDS)
@pytest.mark.parametrize("dtype", [np.float32, BF16])
def test_quantize_bit_exact(built_lib, shape, grid, dtype):
    x = synth(shape, seed=hash((shape, grid)) % 2**31, outliers=0.01, dtype=dtype)
    got = quantize_impl(to_torch(x), grid)
    assert_triple_equal(got, oracle.quantize_impl(x, grid), f"{shape} {grid} {dtype}")


@pytest.mark.parametrize("shape,grid", [((128, 1024), (1, 128)), ((256, 256), (128, 128)), ((32, 64), (4, 4))])
def test_quantize_e5m2_extension(built_lib, shape, grid):
    x = synth(shape, seed=5, scale=1e-3)
    got = quantize_impl(to_torch(x), grid, out_format="e5m2")
    assert_triple_equal(got, oracle.quantize_impl(x, grid, out_format="e5m2"), "e5m2")


def test_distributions_and_edge_values(built_lib):
    shape, grid = (256, 2048), (1, 128)
    cases = {
        "student_t": synth(shape, 11, dist="student_t", outliers=0),
        "tiny": synth(shape, 12, scale=1e-9),             # exercises the 1e-7 floor
        "huge": synth(shape, 13, scale=1e30),
        "weights": synth(shape, 14, scale=0.02, outliers=0),
        "grads": synth(shape, 15, scale=1e-3, outliers=0),
    }
    z = synth(shape, 16)
    z[::2] = 0.0                                          # all-zero super-groups
    z[1, :128] = -0.0
    z[3, 5] = -0.0
    cases["zeros"] = z
    p2 = np.zeros(shape, np.float32)
    p2[:, ::128] = 8.0
    p2[:, 128::256] = np.nextafter(np.float32(8.0), np.float32(0))
    p2[:, 1::128] = np.float32(17.03) / 16
    cases["pow2"] = p2
    for name, x in cases.items():
        for dt in (np.float32, BF16):
            xx = x.astype(dt)
            assert_triple_equal(quantize_impl(to_torch(xx), grid), oracle.quantize_impl(xx, grid), f"{name} {dt}")
        assert_triple_equal(quantize_impl(to_torch(x[:, :256].copy()), (128, 128)),
                            oracle.quantize_impl(x[:, :256].copy(), (128, 128)), f"{name} 128x128")


def test_rank_promotion_and_batching(built_lib):
    v = synth((96,), 21)
    assert_triple_equal(quantize_impl(to_torch(v), (1, 16)), oracle.quantize_impl(v, (1, 16)), "1-D")
    s = np.float32(-2.0)
    got = quantize_impl(torch.tensor(-2.0, device="cuda"), (1, 1))
    assert_triple_equal(got, oracle.quantize_impl(s, (1, 1)), "0-D")
    x3 = synth((3, 16, 1024), 22)
    x3[1] *= 100
    assert_triple_equal(quantize_impl(to_torch(x3), (1, 128)), oracle.quantize_nd(x3, (1, 128)), "3-D fast")
    assert_triple_equal(quantize_impl(to_torch(x3), (16, 128)), oracle.quantize_nd(x3, (16, 128)), "3-D generic")
    x4 = synth((2, 3, 8, 64), 23)
    assert_triple_equal(quantize_impl(to_torch(x4), (4, 16)), oracle.quantize_impl(x4, (4, 16)), "4-D")


@pytest.mark.parametrize("shape,grid", GRIDS)
@pytest.mark.parametrize("out_dtype", ["f32", "bf16"])
def test_dequantize_bit_exact(built_lib, shape, grid, out_dtype):
    x = synth(shape, seed=77, outliers=0.01)
    q, s8, s32 = oracle.quantize_impl(x, grid)
    np_dt, t_dt = (np.float32, torch.float32) if out_dtype == "f32" else (BF16, torch.bfloat16)
    want = oracle.dequantize_impl(q, s8, s32, np_dt, grid)
    tq = torch.from_numpy(bytes_of(q).copy()).cuda().view(torch.float8_e4m3fn)
    t8 = torch.from_numpy(s8.copy()).cuda().view(torch.float8_e8m0fnu)
    got = from_torch(dequantize_impl(tq, t8, to_torch(s32), t_dt, grid))
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_dequantize_negated_scale_and_bwd(built_lib):
    x = synth((64, 1024), 31)
    q, s8, s32 = oracle.quantize_impl(x, (1, 128))
    tq = torch.from_numpy(bytes_of(q).copy()).cuda().view(torch.float8_e4m3fn)
    t8 = torch.from_numpy(s8.copy()).cuda().view(torch.float8_e8m0fnu)
    got = from_torch(dequantize_impl(tq, t8, to_torch(-s32), torch.float32, (1, 128)))
    assert np.array_equal(got, oracle.dequantize_impl(q, s8, -s32, np.float32, (1, 128)))
    g = synth((64, 1024), 32, scale=1e-3, outliers=0)
    for dt in (np.float32, BF16):
        gg = g.astype(dt)
        got = from_torch(dequantize_impl_bwd(t8, to_torch(s32), to_torch(gg), (1, 128)))
        want = oracle.dequantize_impl_bwd(s8, s32, gg, (1, 128))
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_full_size_round_trip_properties(built_lib):
    """Largest benchmark activation: checks size-independent properties instead of the oracle."""
    torch.manual_seed(0)
    x = torch.randn(32768, 2048, device="cuda", dtype=torch.bfloat16)
    q, s8, s32 = quantize_impl(x, (1, 128))
    assert q.view(torch.uint8).bitwise_and(0x7F).max().item() <= 0x78          # |code| <= 256
    amax = x.float().abs().view(-1, 1024).amax(dim=1)
    assert torch.equal(s32.view(-1), amax)                                     # fp32 scale is the super-group amax
    assert s8.view(torch.uint8).max().item() <= 127
    back = dequantize_impl(q, s8, s32, torch.float32, (1, 128))
    scale = (s8.view(torch.uint8).to(torch.int32) << 23).view(torch.float32).view(-1, 8) * s32.view(-1, 1) / 128
    v = x.float().view(-1, 8, 128) / scale.unsqueeze(-1)
    err = (back.view(-1, 8, 128) / scale.unsqueeze(-1) - v).abs()
    # bf16 rounding (2^-9 relative) followed by e4m3 rounding (2^-4 relative, 2^-10 absolute below 2^-6)
    bound = torch.where(v.abs() >= 2.0 ** -6, (2.0 ** -4 + 2.0 ** -8) * v.abs(), 2.0 ** -10 + 2.0 ** -8 * v.abs())
    assert bool((err <= bound).all())
    # a row shard reproduces the bytes of the full tensor (no exchange between shards)
    qs, s8s, s32s = quantize_impl(x[4096:8192].contiguous(), (1, 128))
    assert torch.equal(qs.view(torch.uint8), q[4096:8192].view(torch.uint8))
    assert torch.equal(s8s.view(torch.uint8), s8.view(torch.uint8)[4096 * 2:8192 * 2])


def test_hoisted_division_matches_ieee(diag_lib):
    """The device self-check lives in the diagnostics build of the library (same quantizer sources)."""
    bad = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert diag_lib.pb_debug_division_check(1 << 28, 1234, bad.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    assert bad.item() == 0


def test_errors_raise(built_lib):
    x = torch.zeros(10, 10, device="cuda")
    with pytest.raises(ValueError):
        quantize_impl(x, (4, 4))
    with pytest.raises(RuntimeError):
        quantize_impl(torch.zeros(8, 8), (1, 8))      # CPU tensor: no CPU path
