"""QArrayImpl / qx / Linear on the GPU against compositions of the oracle's functions that follow
pratchya/_qualia/_qarr.py and _qual.py line by line (dequantize -> op -> quantize on the rule's grid)."""
import numpy as np
import pytest
import torch

from helpers import BF16, assert_triple_equal, bytes_of, from_torch, oracle, synth, to_torch
from pratchya_b200 import QArrayImpl, qx
from pratchya_b200._nnx_impl import Linear, LowRankFFN
from pratchya_b200._qualia import fp8_matmul

pytestmark = pytest.mark.gpu


def triple_of(q: QArrayImpl):
    return q.get_value(), q.sc_fp8, q.sc_fp32


def oq(x, grid):
    return oracle.quantize_nd(np.asarray(x, dtype=np.float32), grid)


def odq(t, grid, dtype=np.float32):
    return oracle.dequantize_nd(*t, dtype, grid)


def test_constructor_properties_and_pytree(built_lib):
    x = synth((64, 256), 1)
    q = QArrayImpl(to_torch(x), (16, 16))
    assert q.shape == (64, 256) and q.size == 64 * 256 and q.tgrid == (16, 16) and q.dtype == torch.float8_e4m3fn
    assert_triple_equal(triple_of(q), oq(x, (16, 16)), "ctor")
    children, aux = q.tree_flatten()
    assert aux == (True, (16, 16)) and len(children) == 3
    q2 = QArrayImpl.tree_unflatten(aux, children)
    assert np.array_equal(from_torch(q2.astype(torch.float32)), odq(oq(x, (16, 16)), (16, 16)))
    box = QArrayImpl(to_torch(x), quant=False)
    assert box.tree_flatten()[1] == (False, None) and box.astype(torch.float32).shape == (64, 256)
    copy = QArrayImpl(q)
    assert copy.tgrid == q.tgrid and copy.get_value() is q.get_value()
    # bf16 input is widened to f32 first (exact), 3-D input is quantized per leading index
    x3 = synth((3, 8, 256), 2)
    x3[1] *= 50
    assert_triple_equal(triple_of(QArrayImpl(to_torch(x3.astype(BF16)), (1, 128))), oq(x3.astype(BF16).astype(np.float32), (1, 128)), "3-D bf16")


def test_neg_abs_astype(built_lib):
    x = synth((32, 128), 3)
    q = QArrayImpl(to_torch(x), (1, 16))
    base = odq(oq(x, (1, 16)), (1, 16))
    assert np.array_equal(from_torch((-q).astype(torch.float32)), -base)
    assert np.array_equal(from_torch(abs(q).astype(torch.float32)), np.abs(base))
    assert np.array_equal(from_torch(q.astype(torch.bfloat16)).view(np.uint16), odq(oq(x, (1, 16)), (1, 16), BF16).view(np.uint16))
    assert np.array_equal(from_torch(q.__jax_array__()), base)


@pytest.mark.parametrize("op", ["add", "sub", "mul", "truediv", "floordiv", "mod", "pow"])
def test_elementwise_same_grid(built_lib, op):
    x, y = synth((32, 64), 4, outliers=0), np.abs(synth((32, 64), 5, outliers=0)) + 0.5
    if op == "pow":
        x = np.abs(x) + 0.5
    grid = (4, 16)
    qx_, qy_ = QArrayImpl(to_torch(x), grid), QArrayImpl(to_torch(y), grid)
    fn = {"add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b, "truediv": lambda a, b: a / b,
          "floordiv": lambda a, b: a // b, "mod": lambda a, b: a % b, "pow": lambda a, b: a ** b}[op]
    got = fn(qx_, qy_)
    want_f32 = oracle.elementwise_impl(op, *oq(x, grid), *oq(y, grid), grid)
    got_f32 = from_torch(got.astype(torch.float32))
    want = odq(oq(want_f32, grid), grid)
    # the f32 op itself may differ by an ulp between torch and numpy (pow, division): compare after re-quantization loosely
    assert got.tgrid == grid
    assert np.allclose(got_f32, want, rtol=0.13, atol=np.abs(want).max() * 2 ** -7)
    if op in ("add", "sub", "mul"):
        assert_triple_equal(triple_of(got), oq(want_f32, grid), op)


def test_mixed_operands_return_plain_arrays(built_lib):
    x = synth((16, 64), 6)
    q = QArrayImpl(to_torch(x), (1, 16))
    base = odq(oq(x, (1, 16)), (1, 16))
    dense = to_torch(synth((16, 64), 7))
    out = q + dense
    assert isinstance(out, torch.Tensor) and np.array_equal(from_torch(out), base + from_torch(dense))
    out = 2.0 * q
    assert isinstance(out, torch.Tensor) and np.array_equal(from_torch(out), base * np.float32(2.0))
    out = 1.0 - q
    assert np.array_equal(from_torch(out), np.float32(1.0) - base)
    # different grids: f32 op, quantized on self's grid (_qarr.py:126-127)
    other = QArrayImpl(to_torch(x), (4, 4))
    got = q + other
    want = oq(base + odq(oq(x, (4, 4)), (4, 4)), (1, 16))
    assert got.tgrid == (1, 16)
    assert_triple_equal(triple_of(got), want, "different grids")


def test_getitem_reshape_transpose_sum_concat_at(built_lib):
    x = synth((8, 32, 64), 8)
    q = QArrayImpl(to_torch(x), (16, 16))
    base = odq(oq(x, (16, 16)), (16, 16))
    got = q[2]
    assert got.tgrid == (16, 16)
    assert_triple_equal(triple_of(got), oq(base[2], (16, 16)), "getitem")
    got = q[:, :, 5]
    assert got.tgrid == oracle.adapt_grid((16, 16), (8, 32))
    assert_triple_equal(triple_of(got), oq(base[:, :, 5], got.tgrid), "getitem column")
    got = q.reshape(8, 2048)
    assert got.tgrid == (8, 16)
    assert_triple_equal(triple_of(got), oq(base.reshape(8, 2048), (8, 16)), "reshape")
    q2 = QArrayImpl(to_torch(x[0]), (16, 4))
    b2 = odq(oq(x[0], (16, 4)), (16, 4))
    assert q2.T.tgrid == (4, 16)
    assert_triple_equal(triple_of(q2.T), oq(np.ascontiguousarray(b2.T), (4, 16)), "T")
    assert_triple_equal(triple_of(q2.mT), oq(np.ascontiguousarray(b2.T), (4, 16)), "mT")
    got = q2.transpose(1, 0)
    assert got.tgrid == oracle.adapt_grid((16, 4), (64, 32))
    got = q2.sum(axis=0)
    assert got.shape == (64,) and got.tgrid == oracle.adapt_grid((16, 4), (64,))
    # the f32 reduction order differs between the device and numpy: compare values, not bytes
    want = odq(oq(b2.sum(axis=0), got.tgrid), got.tgrid)
    assert np.allclose(from_torch(got.astype(torch.float32)), want, rtol=0.13, atol=np.abs(want).max() * 2 ** -7)
    cat = QArrayImpl.concat([q2, q2], axis=0)
    assert cat.shape == (64, 64) and cat.tgrid == (16, 4)
    assert_triple_equal(triple_of(cat), oq(np.concatenate([b2, b2], 0), (16, 4)), "concat")
    upd = q2.at[3].set(torch.zeros(64, device="cuda"))
    ref = b2.copy(); ref[3] = 0
    assert_triple_equal(triple_of(upd), oq(ref, (16, 4)), "at.set")
    ap = q2.apply(lambda v: v * 2.0)
    assert_triple_equal(triple_of(ap), oq(b2 * np.float32(2), (16, 4)), "apply")


def test_qx_dispatcher(built_lib):
    x = synth((16, 64), 9)
    q = QArrayImpl(to_torch(x), (1, 16))
    base = odq(oq(x, (1, 16)), (1, 16))
    got = qx.tanh(q)                                        # same shape: re-quantized on the gcd grid
    assert isinstance(got, QArrayImpl) and got.tgrid == (1, 16)
    want = oq(np.tanh(base), (1, 16))
    assert np.allclose(from_torch(got.astype(torch.float32)), odq(want, (1, 16)), rtol=0.13, atol=2 ** -9)
    got = qx.sum(q)                                         # shape changed: unquantized box
    assert isinstance(got, QArrayImpl) and not got._is_quantized()
    assert np.allclose(got.get_value().item(), base.sum(), rtol=1e-5)
    got = qx.relu(to_torch(x))                              # no quantized input: unquantized box
    assert not got._is_quantized()
    with pytest.raises(AttributeError):
        qx.no_such_function


def test_matmul_operator_and_fp8_matmul(built_lib):
    x, w = synth((256, 1024), 10), synth((1024, 256), 11, scale=0.02, outliers=0)
    qa, qw = QArrayImpl(to_torch(x), (1, 128)), QArrayImpl(to_torch(w), (128, 128))
    y = qa @ qw                                             # tensor-core path, result re-quantized on (1,128)
    assert isinstance(y, QArrayImpl) and y.tgrid == (1, 128) and y.shape == (256, 256)
    ref = oracle.matmul_impl(*oq(x, (1, 128)), *oq(w, (128, 128)), (1, 128), (128, 128), acc=np.float64)
    got = from_torch(y.astype(torch.float32))
    assert np.abs(got - ref).max() <= (2 ** -4 + 2 ** -7) * np.abs(ref).max()      # fp8 re-quantization of the output
    dense = to_torch(synth((1024, 64), 12))
    out = qa @ dense                                        # mixed: plain f32 array
    want = oracle.matmul_mixed_impl(*oq(x, (1, 128)), from_torch(dense), (1, 128))
    assert isinstance(out, torch.Tensor) and np.allclose(from_torch(out), want, rtol=1e-4, atol=1e-3)
    out = to_torch(synth((8, 256), 13)) @ qa                # reflected mixed
    assert isinstance(out, torch.Tensor) and out.shape == (8, 1024)
    a, b = synth((32, 64), 14), synth((64, 48), 15)
    got = from_torch(fp8_matmul(to_torch(a), to_torch(b), (1, 16)))
    want = oracle.fp8_matmul(a, b, (1, 16))
    assert np.allclose(got, want, rtol=0.14, atol=np.abs(want).max() * 2 ** -6)


def test_linear_layers(built_lib):
    x = synth((4, 64, 1024), 16).astype(BF16)
    w = synth((1024, 512), 17, scale=0.02, outliers=0)
    layer = Linear(1024, 512, (128, 128), kernel=to_torch(w))
    y = layer(to_torch(x))                                  # (Q(x,(1,128)) @ W).astype(bf16): fake-quantized output
    assert y.shape == (4, 64, 512) and y.dtype == torch.bfloat16
    want = oracle.linear_forward(x, oq(w, (128, 128)), (128, 128)).astype(np.float32)
    got = from_torch(y).astype(np.float32)
    assert np.abs(got - want).max() <= 2 ** -3 * np.abs(want).max()
    ym = layer.matmul(to_torch(x), out_dtype=torch.float32)  # the same product without the final fake-quantization
    ref = oracle.matmul_impl(*oracle.quantize_nd(x.astype(np.float32), (1, 128)), *oq(w, (128, 128)), (1, 128), (128, 128), acc=np.float64)
    assert np.abs(from_torch(ym) - ref).max() <= 1e-2 * np.abs(ref).max()
    ffn = LowRankFFN(256, 32, (16, 16), generator=torch.Generator(device="cuda").manual_seed(0))
    out = ffn(to_torch(synth((8, 256), 18)))
    assert out.shape == (8, 256) and torch.isfinite(out).all()
    assert ffn.down.kernel.tgrid == (16, 1) and ffn.up.kernel.tgrid == (16, 1)


@pytest.mark.parametrize("grid,shape", [((1, 128), (64, 1024)), ((128, 128), (256, 384)), ((16, 16), (48, 80)), ((1, 16), (3, 8, 64)),
                                        ((4, 4), (12, 20))])
def test_fused_elementwise_has_the_bits_of_the_three_steps(built_lib, grid, shape):
    """add / sub / mul / div of two quantized arrays in one kernel against dequantize, dequantize, op."""
    from helpers import synth, to_torch
    from pratchya_b200._qualia import _ops, dequantize_impl, quantize_impl
    x = synth(shape, seed=1, outliers=0.02)
    y = synth(shape, seed=2, outliers=0.02)
    y.reshape(-1)[:7] = 0.0                     # division by zero and 0/0
    x.reshape(-1)[:3] = 0.0
    xq, yq = quantize_impl(to_torch(x), grid), quantize_impl(to_torch(y), grid)
    xd, yd = dequantize_impl(*xq, torch.float32, grid), dequantize_impl(*yq, torch.float32, grid)
    for impl, op in ((_ops.add_impl, torch.add), (_ops.sub_impl, torch.sub), (_ops.mul_impl, torch.mul), (_ops.truediv_impl, torch.div)):
        got = impl(*xq, *yq, grid)
        want = op(xd, yd)
        assert got.shape == want.shape and got.dtype == torch.float32
        same = (got.view(torch.int32) == want.view(torch.int32)) | (torch.isnan(got) & torch.isnan(want))
        assert bool(same.all()), f"{op.__name__} on grid {grid}: {(~same).sum().item()} elements differ"
