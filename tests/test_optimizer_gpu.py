"""GPU parity of the optimizer's quantized-momentum step (pb_momentum_update) with the oracle's
restatement of pratchya/_nnx_impl/_optimizer.py:171-205 and with the literal sequence of calls
(dequantize, dequantize, blend, blend, quantize).  Bit-exact: everything is f32 multiplies, adds and
the quantizer's arithmetic."""
import numpy as np
import pytest
import torch

from helpers import assert_triple_equal, bytes_of, from_torch, oracle, synth, to_torch
from pratchya_b200 import QArrayImpl
from pratchya_b200._nnx_impl import lion_update, momentum_update
from pratchya_b200._qualia import dequantize_impl, quantize_impl

pytestmark = pytest.mark.gpu


def np_triple(q):
    return (bytes_of(q.get_value()), bytes_of(q.sc_fp8), from_torch(q.sc_fp32))


@pytest.mark.parametrize("shape,grid", [((256, 384), (128, 128)), ((2048, 2048), (128, 128)), ((64, 256), (1, 128)), ((48, 80), (16, 16)),
                                        ((3, 128, 8), (128, 1)), ((12, 20), (4, 4))])
@pytest.mark.parametrize("beta1,beta2", [(0.9, 0.99), (0.95, 0.98)])
def test_momentum_step_matches_oracle_and_literal_calls(built_lib, shape, grid, beta1, beta2):
    g = synth(shape, seed=11, scale=1e-3, outliers=0.01)
    m = synth(shape, seed=12, scale=5e-4, outliers=0)
    m.reshape(-1)[: m.size // 3] = 0.0              # a young momentum: many zero blocks
    gq, mq = QArrayImpl(to_torch(g), grid), QArrayImpl(to_torch(m), grid)
    c, new_m = momentum_update(gq, mq, beta1, beta2)
    # the oracle on the same quantized inputs
    quant = oracle.quantize_nd if len(shape) == 3 else oracle.quantize_impl
    og = quant(np.asarray(g), grid)
    om = quant(np.asarray(m), grid)
    if len(shape) == 3:
        gd, md = oracle.dequantize_nd(*og, np.float32, grid), oracle.dequantize_nd(*om, np.float32, grid)
        b1, c1, b2, c2 = np.float32(beta1), np.float32(1.0 - beta1), np.float32(beta2), np.float32(1.0 - beta2)
        oc = b1 * md + c1 * gd
        onm = oracle.quantize_nd((b2 * md + c2 * gd).astype(np.float32), grid)
    else:
        oc, onm = oracle.momentum_update(og, om, grid, beta1, beta2)
    assert np.array_equal(c.cpu().numpy().view(np.uint32), np.asarray(oc, dtype=np.float32).view(np.uint32)), "c differs from the oracle"
    assert_triple_equal(np_triple(new_m), (onm[0].view(np.uint8), onm[1].view(np.uint8), onm[2]), "new momentum vs oracle")
    # the literal sequence on the GPU
    gd = dequantize_impl(gq.get_value(), gq.sc_fp8, gq.sc_fp32, torch.float32, grid)
    md = dequantize_impl(mq.get_value(), mq.sc_fp8, mq.sc_fp32, torch.float32, grid)
    f = lambda v: float(np.float32(v))
    want_c = f(beta1) * md + f(1.0 - beta1) * gd
    want_m = quantize_impl(f(beta2) * md + f(1.0 - beta2) * gd, grid)
    assert torch.equal(c, want_c)
    assert_triple_equal(np_triple(new_m), (bytes_of(want_m[0]), bytes_of(want_m[1]), from_torch(want_m[2])), "new momentum vs literal calls")


def test_lion_update_and_rejections(built_lib):
    p = to_torch(synth((128, 128), seed=1))
    c = to_torch(synth((128, 128), seed=2))
    u = lion_update(c, p, 1e-3, 0.1)
    assert torch.equal(u, -(1e-3 * torch.sign(c) + 1e-3 * 0.1 * p))
    a = QArrayImpl(p, (128, 128))
    b = QArrayImpl(p, (1, 128))
    with pytest.raises(ValueError):
        momentum_update(a, b, 0.9, 0.99)


@pytest.mark.parametrize("shape,grid", [((24, 2048, 2048), (128, 128)), ((4, 256, 384), (128, 128)), ((3, 64, 256), (1, 128)), ((5, 48, 80), (16, 16)),
                                        ((2, 128, 8), (128, 1))])
def test_stacked_momentum_step_is_the_bf16_scan_of_the_reference(built_lib, shape, grid):
    """pb_momentum_update_stacked against the oracle's restatement of the scanned branch for stacked parameters
    (pratchya/_nnx_impl/_optimizer.py:108-160): bf16 dequantization, bf16 blend, re-quantization per layer.  Bit-exact:
    c as bf16 bits, the new momentum as its triple."""
    from pratchya_b200._nnx_impl import momentum_update_stacked
    beta1, beta2 = 0.9, 0.99
    gen = torch.Generator(device="cuda").manual_seed(5)
    g = torch.randn(shape, device="cuda", generator=gen) * 1e-3
    m = torch.randn(shape, device="cuda", generator=gen) * 5e-4
    m[0, : shape[1] // 2] = 0.0                       # a young momentum: zero blocks
    gq, mq = QArrayImpl(g, grid), QArrayImpl(m, grid)
    assert gq.sc_fp32.shape[0] == shape[0]            # quantized per layer
    c, new_m = momentum_update_stacked(gq, mq, beta1, beta2)
    assert c.dtype == torch.bfloat16 and tuple(c.shape) == shape
    og = tuple(np.asarray(t) for t in np_triple(gq))
    om = tuple(np.asarray(t) for t in np_triple(mq))
    og = (og[0].view(oracle.E4M3), og[1], og[2])
    om = (om[0].view(oracle.E4M3), om[1], om[2])
    layers = range(shape[0]) if shape[0] <= 6 else (0, 7, 23)       # the large stack: three of its layers on the CPU
    for i in layers:
        oc, onm = oracle.momentum_update_stacked(tuple(t[i:i + 1] for t in og), tuple(t[i:i + 1] for t in om), grid, beta1, beta2)
        assert np.array_equal(from_torch(c[i]).view(np.uint16), oc[0].view(np.uint16)), f"layer {i}: c differs from the oracle"
        got = (bytes_of(new_m.get_value()[i]), bytes_of(new_m.sc_fp8[i]), from_torch(new_m.sc_fp32[i]))
        assert_triple_equal(got, (onm[0][0].view(np.uint8), onm[1][0].view(np.uint8), onm[2][0]), f"layer {i}: new momentum vs oracle")
    with pytest.raises(ValueError):
        momentum_update_stacked(QArrayImpl(g[0], grid), QArrayImpl(m[0], grid), beta1, beta2)
