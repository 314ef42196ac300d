"""Known answers derived by hand from the reference rule (pratchya/_qualia/_qarr.py:458-506,
:541-569) pin the CPU oracle.  The reference itself ships no test vectors."""
import ml_dtypes
import numpy as np
import pytest

from oracle import qarr_oracle as o

E4M3 = ml_dtypes.float8_e4m3fn


def u8(a):
    return np.ascontiguousarray(a).view(np.uint8)


def test_all_zero_group():
    q, s8, s32 = o.quantize_impl(np.zeros((4, 4), np.float32), (4, 4))
    assert (u8(q) == 0).all() and s8.tolist() == [[0]] and s32.tolist() == [[[0.0]]]
    assert (o.dequantize_impl(q, s8, s32, np.float32, (4, 4)) == 0).all()


@pytest.mark.parametrize("c", [3.5, -3.5, 1e-3, 12345.0])
def test_constant_block_alone_in_group(c):
    x = np.full((1, 16), c, np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 16))          # a*b//16 = 1 -> K = 1
    assert (u8(q) == (0x70 if c > 0 else 0xF0)).all()  # +-128
    assert s8.tolist() == [[127]] and s32[0, 0, 0] == np.float32(abs(c))
    assert np.array_equal(o.dequantize_impl(q, s8, s32, np.float32, (1, 16)), x)


def test_grid_1x1_is_per_element():
    x = np.array([[2.0, -0.25], [7.0, 0.0]], np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 1))
    assert u8(q).tolist() == [[0x70, 0xF0], [0x70, 0x00]]
    assert s8.reshape(-1).tolist() == [127, 127, 127, 0]
    assert s32.reshape(-1).tolist() == [2.0, 0.25, 7.0, 0.0]


def test_scalar_and_vector_rank_promotion():
    q, s8, s32 = o.quantize_impl(np.float32(-2.0), (1, 1))
    assert q.shape == () and s8.shape == (1, 1) and s32.shape == (1, 1, 1) and u8(q).item() == 0xF0
    q, s8, s32 = o.quantize_impl(np.arange(32, dtype=np.float32), (1, 16))
    assert q.shape == (32,) and s8.shape == (2, 1) and s32.shape == (2, 1, 1)


def test_power_of_two_ratio_between_blocks():
    # grid (1,32): a*b//16 = 2 -> two blocks share one fp32 amax.
    x = np.zeros((1, 64), np.float32)
    x[0, 0] = 8.0          # block 0 amax = M_j
    x[0, 1] = 3.0          # 3/8*128 = 48 = 1.5*2^5 -> 0x64
    x[0, 32] = 0.5         # block 1 amax = M_j * 2^-4 -> e8m0 127-4, element -> 128
    x[0, 33] = -0.25       # -0.25/0.5*128 = -64 -> 0xE8
    q, s8, s32 = o.quantize_impl(x, (1, 32))
    assert s8.tolist() == [[127, 123]] and s32.reshape(-1).tolist() == [8.0]
    b = u8(q)[0]
    assert b[0] == 0x70 and b[1] == 0x64 and b[32] == 0x70 and b[33] == 0xE8
    assert np.array_equal(o.dequantize_impl(q, s8, s32, np.float32, (1, 32)), x)


def test_block_amax_between_powers_lands_in_128_256():
    x = np.zeros((1, 64), np.float32)
    x[0, 0] = 8.0
    x[0, 32] = 0.75        # 0.09375 = 1.5*2^-4 -> e8m0 123, S_eff = 0.5, value 192 = 1.5*2^7 -> 0x74
    q, s8, _ = o.quantize_impl(x, (1, 32))
    assert s8.tolist() == [[127, 123]] and u8(q)[0, 32] == 0x74


def test_largest_code_is_256():
    x = np.zeros((1, 64), np.float32)
    x[0, 0] = 8.0
    x[0, 32] = np.nextafter(np.float32(8.0), np.float32(0.0))   # ratio just below 1 -> e8m0 126 -> ~255.99998 -> 256
    q, s8, _ = o.quantize_impl(x, (1, 32))
    assert s8.tolist() == [[127, 126]] and u8(q)[0, 32] == 0x78


def test_double_rounding_through_bf16():
    # v = 17.03: bf16 (spacing 0.125) -> 17.0, then the e4m3 tie 17 -> 16 (even); a direct cast gives 18.
    x = np.zeros((1, 16), np.float32)
    x[0, 0] = 1.0
    x[0, 1] = np.float32(17.03) / np.float32(128.0)
    q, _, _ = o.quantize_impl(x, (1, 16))
    assert u8(q)[0, 1] == 0x58
    assert u8((x[0, 1:2] * np.float32(128)).astype(E4M3))[0] == 0x59


def test_negative_zero_keeps_its_sign():
    x = np.array([[1.0, -0.0, 0.0, -1e-30]], np.float32)
    q, _, _ = o.quantize_impl(x, (1, 4))
    assert u8(q)[0].tolist() == [0x70, 0x80, 0x00, 0x80]


def test_scale_floor_is_only_on_the_quantize_side():
    x = np.full((1, 16), 1e-9, np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 16))
    # S_eff = max(1e-9, 1e-7) = 1e-7 -> 1.28 -> bf16 1.28125 -> e4m3 1.25 = 0x3A
    assert (u8(q) == 0x3A).all() and s8.tolist() == [[127]] and s32[0, 0, 0] == np.float32(1e-9)
    back = o.dequantize_impl(q, s8, s32, np.float32, (1, 16))
    assert np.allclose(back, 1.25 * 1e-9 / 128, rtol=1e-6)      # not the input: reference behaviour


def test_supergroup_is_eight_row_major_blocks_for_1x128():
    # [2, 1024] on (1,128): 16 blocks, K = 8 -> one fp32 amax per row here
    x = np.ones((2, 1024), np.float32)
    x[1] *= 4
    q, s8, s32 = o.quantize_impl(x, (1, 128))
    assert s8.shape == (2, 8) and s32.reshape(-1).tolist() == [1.0, 4.0] and (u8(q) == 0x70).all()
    # [4, 512]: K = 8 spans two rows
    x = np.ones((4, 512), np.float32)
    x[1] *= 4
    q, s8, s32 = o.quantize_impl(x, (1, 128))
    assert s32.reshape(-1).tolist() == [4.0, 1.0]
    assert s8.tolist() == [[125] * 4 + [127] * 4, [127] * 8]


def test_supergroup_of_128x128_weight_is_tensor_wide_up_to_1024_blocks():
    assert o.group_geometry(2048, 8192, (128, 128)) == (1, 1024)
    assert o.group_geometry(2048, 2048, (128, 128)) == (1, 256)
    assert o.group_geometry(4096, 16384, (128, 128)) == (4, 1024)
    assert o.group_geometry(8192, 2048, (1, 128)) == (16384, 8)
    assert o.group_geometry(2048, 2048, (128, 1)) == (4096, 8)


def test_three_dim_values_are_quantized_per_leading_index():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 8, 64)).astype(np.float32)
    x[1] *= 100
    q, s8, s32 = o.quantize_nd(x, (4, 16))
    for i in range(3):
        qi, s8i, s32i = o.quantize_impl(x[i], (4, 16))
        assert np.array_equal(u8(q[i]), u8(qi)) and np.array_equal(s8[i], s8i) and np.array_equal(s32[i], s32i)


def test_negation_flips_only_the_fp32_scale():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((8, 64)).astype(np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 16))
    a = o.dequantize_impl(q, s8, -s32, np.float32, (1, 16))
    b = o.dequantize_impl(q, s8, s32, np.float32, (1, 16))
    assert np.array_equal(a, -b)


def test_nan_e8m0_cotangent_is_replaced_by_one():
    q = np.array([[64.0]], np.float32).astype(E4M3)
    got = o.quantize_impl_bwd((q, np.array([[0xFF]], np.uint8), np.array([[[2.0]]], np.float32)), (1, 1))
    assert got.tolist() == [[64.0 * 1.0 * 2.0 / 128.0]]
    dense = np.ones((2, 2), np.float32)
    assert o.quantize_impl_bwd(dense, (1, 1)) is dense


def test_round_trip_error_bound():
    # |q - v| <= (2^-4 + 2^-9)|v| for |v| >= 2^-6, <= 2^-10 below (bf16 then e4m3 rounding)
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 1024)).astype(np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 128))
    scale = np.repeat(o.effective_scale(s8, s32).reshape(64, 8), 128, axis=1)
    v = x / scale
    err = np.abs(q.astype(np.float32) - v)
    bound = np.where(np.abs(v) >= 2.0 ** -6, (2.0 ** -4 + 2.0 ** -8) * np.abs(v), 2.0 ** -10 + 2.0 ** -8 * np.abs(v))
    assert (err <= bound).all()


def test_row_shard_invariance():
    # a row shard whose block count is a multiple of 8 quantizes to the same bytes as the full tensor
    rng = np.random.default_rng(3)
    x = rng.standard_normal((32, 1024)).astype(np.float32)
    q, s8, s32 = o.quantize_impl(x, (1, 128))
    for lo, hi in [(0, 16), (16, 32), (8, 24)]:
        qs, s8s, s32s = o.quantize_impl(x[lo:hi], (1, 128))
        assert np.array_equal(u8(qs), u8(q[lo:hi])) and np.array_equal(s8s, s8[lo:hi]) and np.array_equal(s32s, s32[lo:hi])


def test_adapt_grid_rule():
    assert o.adapt_grid((128, 128), (2048, 96)) == (128, 32)
    assert o.adapt_grid((1, 128), (7,)) == (1, 1)
    assert o.adapt_grid((16, 16), ()) == (1, 1)


def test_matmul_and_linear_shapes():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((16, 256)).astype(np.float32)
    w = (rng.standard_normal((256, 128)) * 0.02).astype(np.float32)
    wq = o.quantize_impl(w, (128, 128))
    y = o.linear_forward(x, wq, (128, 128))
    ref = x @ w
    assert y.shape == (16, 128) and np.abs(y - ref).max() < 0.1 * np.abs(ref).max()
    (gx, gw) = o.matmul_impl_bwd((*o.quantize_impl(x, (1, 128)), *wq), np.ones((16, 128), np.float32), (1, 128), (128, 128))
    assert gx[0].shape == (16, 256) and gw[0].shape == (256, 128)
    fx, fy = o.fp8_matmul_bwd(x, w, np.ones((16, 128), np.float32), (1, 16))
    assert fx.shape == x.shape and fy.shape == w.shape


def test_momentum_update_known_answers():
    """_optimizer.py:171-205 restated: constant g and m on one (4,4) block dequantize exactly, so c and
    new_m are the scalar blends, and new_m re-quantizes to the byte of 128 with its own value as sc32."""
    import numpy as np
    from oracle import qarr_oracle as o
    g = np.full((4, 4), 2.0, np.float32)
    m = np.full((4, 4), -1.0, np.float32)
    gq, mq = o.quantize_impl(g, (4, 4)), o.quantize_impl(m, (4, 4))
    c, nm = o.momentum_update(gq, mq, (4, 4), 0.9, 0.99)
    b1, c1, b2, c2 = np.float32(0.9), np.float32(1.0 - 0.9), np.float32(0.99), np.float32(1.0 - 0.99)
    assert np.all(c == b1 * np.float32(-1.0) + c1 * np.float32(2.0))
    want = np.float32(b2 * np.float32(-1.0) + c2 * np.float32(2.0))
    assert nm[2].reshape(-1)[0] == abs(want)
    assert np.all(nm[0].view(np.uint8) == 0xF0)            # -128 in e4m3
    assert np.all(nm[1].view(np.uint8) == 127)
    # a zero gradient leaves beta2 * m; a zero momentum starts at (1 - beta2) * g
    z = o.quantize_impl(np.zeros((4, 4), np.float32), (4, 4))
    _, nm0 = o.momentum_update(z, mq, (4, 4), 0.9, 0.99)
    assert nm0[2].reshape(-1)[0] == np.float32(b2 * np.float32(1.0))
    _, nm1 = o.momentum_update(gq, z, (4, 4), 0.9, 0.99)
    assert nm1[2].reshape(-1)[0] == np.float32(c2 * np.float32(2.0))


def test_non_finite_inputs_follow_the_rule_s_arithmetic():
    """What the reference's arithmetic gives for non-finite inputs (numpy and jax.numpy agree on these steps: max and
    maximum propagate NaN).  The CUDA kernels depart from it knowingly (their amax reductions drop NaNs; the header
    says so at pb_quantize), so these are answers of the oracle only."""
    x = np.ones((1, 2048), dtype=np.float32)
    x[0, 5] = np.nan                     # first super-group (columns 0..1023)
    x[0, 1500] = np.inf                  # second super-group
    q, s8, s32 = o.quantize_impl(x, (1, 128))
    qb = q.view(np.uint8)
    # a NaN reaches the block amax, the super-group amax and, through S_eff, every element of the super-group
    assert np.isnan(s32[0, 0, 0]) and (qb[0, :1024] & 0x7F == 0x7F).all()
    # an Inf amax: the block holding it has the ratio inf/inf = NaN (scale byte 255, which decodes to Inf: its finite
    # elements become 0 and the Inf itself NaN); the other blocks have the ratio 1/inf = 0, and 0 * inf = NaN in S_eff
    assert np.isinf(s32[1, 0, 0])
    assert s8[0].tolist() == [255] * 8 and s8[1].tolist() == [0, 0, 0, 255, 0, 0, 0, 0]
    blk = qb[0, 1024:].reshape(8, 128)
    assert (blk[[0, 1, 2, 4, 5, 6, 7]] & 0x7F == 0x7F).all()
    assert blk[3, 1500 - 1024 - 384] & 0x7F == 0x7F and np.delete(blk[3], 1500 - 1024 - 384).max() == 0
