"""GPU parity of the two-launch linear step (pb_quantize_for_gemm + pb_gemm_tn_ex) with the
four-launch path it shortens (pb_quantize + pb_gemm_tn) and with the oracle.

Bit-exact: the quantized triple against the oracle's quantize_impl and against pb_quantize, and
the product against pb_gemm_tn on the same triple (same kernel, same scales, so the same bits).
"""
import numpy as np
import pytest
import torch

from helpers import BF16, assert_triple_equal, bytes_of, from_torch, oracle, synth, to_torch
from pratchya_b200 import _lib
from pratchya_b200._nnx_impl import Linear
from pratchya_b200._qualia import LinearStep, matmul_impl, quantize_impl
from pratchya_b200._qualia import _ops

pytestmark = pytest.mark.gpu


def weight(k, n, seed):
    w = synth((k, n), seed=seed, scale=0.02, outliers=0)
    wq = quantize_impl(to_torch(w), (128, 128))
    return wq, _ops.transpose_bytes(wq[0])


def np_triple(t):
    q, s8, s32 = t
    return (bytes_of(q), bytes_of(s8), from_torch(s32))


@pytest.mark.parametrize("m,n,k,dtype", [(256, 1024, 1024, np.float32), (128, 2048, 2048, BF16), (200, 1024, 2048, BF16),
                                         (1000, 2048, 1024, np.float32), (2048, 8192, 2048, BF16)])
def test_step_equals_separate_calls_and_oracle(built_lib, m, n, k, dtype):
    x = synth((m, k), seed=m + k, outliers=0.01).astype(dtype)
    wq, w_t = weight(k, n, seed=n)
    step = LinearStep(w_t, wq[1], wq[2], rows=m, out_dtype=torch.float32)
    xt = to_torch(x)
    for call in range(3):          # first call prepares the weight's scales, later ones reuse them
        d, triple = step(xt)
        _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
        want = quantize_impl(xt, (1, 128))
        assert_triple_equal(np_triple(triple), np_triple(want), f"call {call}: fused quantizer vs pb_quantize")
        ref = matmul_impl(*want, *wq, (1, 128), (128, 128), y_fp8_t=w_t)
        assert torch.equal(d, ref), f"call {call}: two-launch product differs from pb_gemm_tn"
    oq = oracle.quantize_impl(np.asarray(x), (1, 128))
    assert_triple_equal(np_triple(triple), (oq[0].view(np.uint8), oq[1].view(np.uint8), oq[2]), "fused quantizer vs oracle")


def test_step_sees_new_activations_and_refreshed_weight(built_lib):
    m, n, k = 384, 1024, 1024
    wq, w_t = weight(k, n, seed=5)
    step = LinearStep(w_t, wq[1], wq[2], rows=m, out_dtype=torch.bfloat16)
    for seed in (1, 2):
        xt = to_torch(synth((m, k), seed=seed, scale=10.0 ** seed).astype(BF16))
        d, _ = step(xt)
        ref = matmul_impl(*quantize_impl(xt, (1, 128)), *wq, (1, 128), (128, 128), y_fp8_t=w_t, out_dtype=torch.bfloat16)
        assert torch.equal(d, ref)
    # new weight scales in the same buffers: stale until refresh_weight()
    wq2, w_t2 = weight(k, n, seed=6)
    w_t.copy_(w_t2); wq[1].copy_(wq2[1]); wq[2].copy_(wq2[2] * 4)
    step.refresh_weight()
    d, _ = step(xt)
    ref = matmul_impl(*quantize_impl(xt, (1, 128)), wq2[0], wq2[1], wq2[2] * 4, (1, 128), (128, 128), y_fp8_t=w_t2,
                      out_dtype=torch.bfloat16)
    assert torch.equal(d, ref)


def test_linear_matmul_uses_the_step_and_matches(built_lib):
    k, n = 1024, 512
    lin = Linear(k, n, (128, 128), generator=torch.Generator(device="cuda").manual_seed(3))
    x = to_torch(synth((2, 96, k), seed=9))
    y = lin.matmul(x)
    assert lin._steps and all(v is not None for v in lin._steps.values())
    kq = lin.kernel
    ref = matmul_impl(*quantize_impl(x, (1, 128)), kq.get_value(), kq.sc_fp8, kq.sc_fp32, (1, 128), (128, 128))
    assert y.shape == (2, 96, n)
    assert torch.equal(y, ref)


def test_rejections(built_lib):
    wq, w_t = weight(1024, 256, seed=1)
    with pytest.raises(ValueError):
        LinearStep(w_t[:, :512].contiguous(), wq[1], wq[2], rows=128)          # depth 512: not whole super-groups
    step = LinearStep(w_t, wq[1], wq[2], rows=128)
    with pytest.raises(ValueError):
        step(torch.zeros((64, 1024), device="cuda"))
    # unknown flag bits
    xq = quantize_impl(torch.zeros((128, 1024), device="cuda"), (1, 128))
    a = _ops._operand(*xq, 128, 1024, (1, 128))
    d = torch.empty((128, 256), device="cuda")
    st = built_lib.pb_gemm_tn_ex(a, step.b, d.data_ptr(), 0, 256, step.ws.data_ptr(), step.ws_bytes, 8, None)
    assert st == _lib.PB_ERR_UNSUPPORTED
    # a weight whose super-groups do not span eight k-blocks of every row: the fused preparation refuses
    wq3, w_t3 = weight(1024, 384, seed=2)         # 8 x 3 blocks in super-groups of 8: no run of k-blocks shares a factor
    step3 = LinearStep(w_t3, wq3[1], wq3[2], rows=128)
    with pytest.raises(_lib.PbError) as e:
        step3(torch.zeros((128, 1024), device="cuda"))
    assert e.value.status == _lib.PB_ERR_UNSUPPORTED
    # Linear falls back to the four-launch path for such a weight
    lin = Linear(1024, 384, (128, 128), generator=torch.Generator(device="cuda").manual_seed(4))
    x = to_torch(synth((128, 1024), seed=3))
    y = lin.matmul(x)
    assert list(lin._steps.values()) == [None]
    kq = lin.kernel
    assert torch.equal(y, matmul_impl(*quantize_impl(x, (1, 128)), kq.get_value(), kq.sc_fp8, kq.sc_fp32, (1, 128), (128, 128)))


@pytest.mark.parametrize("shape,out_dtype", [((256, 1024), torch.float32), ((3, 64, 2048), torch.bfloat16), ((1000, 8192), torch.bfloat16),
                                             ((8, 1024), torch.float32)])
def test_fake_quantize_has_the_bits_of_quantize_then_dequantize(built_lib, shape, out_dtype):
    from pratchya_b200._qualia import dequantize_impl, fake_quantize_impl
    x = synth(shape, seed=sum(shape), outliers=0.01)
    x.reshape(-1)[:2048] = 0.0            # an all-zero super-group and a half-zero one
    x.reshape(-1)[5000] = -0.0
    xt = to_torch(x)
    got = fake_quantize_impl(xt, (1, 128), out_dtype)
    want = dequantize_impl(*quantize_impl(xt, (1, 128)), out_dtype, (1, 128))
    assert got.dtype == out_dtype and got.shape == want.shape
    assert torch.equal(got.view(torch.int32 if out_dtype == torch.float32 else torch.int16),
                       want.view(torch.int32 if out_dtype == torch.float32 else torch.int16))
    oq = oracle.quantize_nd(np.asarray(x), (1, 128)) if len(shape) == 3 else oracle.quantize_impl(np.asarray(x), (1, 128))
    ref = (oracle.dequantize_nd if len(shape) == 3 else oracle.dequantize_impl)(*oq, np.float32, (1, 128))
    if out_dtype == torch.float32:
        assert np.array_equal(got.cpu().numpy().view(np.uint32), np.asarray(ref, dtype=np.float32).view(np.uint32))


def test_fake_quantize_falls_back_on_other_grids_and_inputs(built_lib):
    from pratchya_b200._qualia import dequantize_impl, fake_quantize_impl
    x = to_torch(synth((256, 256), seed=3))
    for grid in ((128, 128), (1, 16), (16, 16)):
        got = fake_quantize_impl(x, grid, torch.float32)
        assert torch.equal(got, dequantize_impl(*quantize_impl(x, grid), torch.float32, grid))
    xb = to_torch(synth((128, 1024), seed=4).astype(BF16))           # bf16 input: the two-call path
    assert torch.equal(fake_quantize_impl(xb, (1, 128), torch.bfloat16),
                       dequantize_impl(*quantize_impl(xb, (1, 128)), torch.bfloat16, (1, 128)))
    # the C entry point itself refuses what it has no kernel for
    out = torch.empty_like(x)
    st = built_lib.pb_fake_quantize(x.data_ptr(), 0, 1, 256, 256, 128, 128, 0, out.data_ptr(), 0, None)
    assert st == _lib.PB_ERR_UNSUPPORTED


def test_linear_call_equals_the_three_reference_steps(built_lib):
    from pratchya_b200 import QArrayImpl
    k, n = 1024, 2048
    lin = Linear(k, n, (128, 128), generator=torch.Generator(device="cuda").manual_seed(11))
    for x in (to_torch(synth((4, 64, k), seed=1)), to_torch(synth((200, k), seed=2).astype(BF16))):
        got = lin(x)
        want = (QArrayImpl(x, (1, 128)) @ lin.kernel).astype(x.dtype)
        assert got.dtype == x.dtype and got.shape == want.shape
        assert torch.equal(got, want)


@pytest.mark.parametrize("shape,fmt", [((128, 1024), "e4m3"), ((1024, 2048), "e4m3"), ((2, 256, 1024), "e4m3"), ((384, 3072), "e5m2")])
def test_dual_quantizer_equals_the_two_calls(built_lib, shape, fmt):
    from pratchya_b200._qualia import quantize_dual_impl, quantize_transposed_impl
    x = synth(shape, seed=sum(shape), outliers=0.01).astype(BF16)
    x.reshape(-1)[:1024] = 0
    xt = to_torch(x)
    (row, tr) = quantize_dual_impl(xt, out_format=fmt)
    assert_triple_equal(np_triple(row), np_triple(quantize_impl(xt, (1, 128), out_format=fmt)), "row triple")
    assert_triple_equal(np_triple(tr), np_triple(quantize_transposed_impl(xt, 128, out_format=fmt)), "transposed triple")
    if fmt == "e4m3" and len(shape) == 2:
        oq = oracle.quantize_impl(np.ascontiguousarray(np.asarray(x).astype(np.float32).T), (1, 128))
        assert_triple_equal(np_triple(tr), (oq[0].view(np.uint8), oq[1].view(np.uint8), oq[2]), "transposed triple vs oracle on x^T")


def test_dual_quantizer_falls_back(built_lib):
    from pratchya_b200._qualia import quantize_dual_impl, quantize_transposed_impl
    for x in (to_torch(synth((128, 1024), seed=1)),                       # f32 input
              to_torch(synth((128, 512), seed=2).astype(BF16))):          # cols not a multiple of 1024
        row, tr = quantize_dual_impl(x)
        assert_triple_equal(np_triple(row), np_triple(quantize_impl(x, (1, 128))), "row")
        assert_triple_equal(np_triple(tr), np_triple(quantize_transposed_impl(x, 128)), "transposed")
    x = to_torch(synth((128, 512), seed=2).astype(BF16))
    outs = [torch.empty(128 * 512, dtype=torch.uint8, device="cuda") for _ in range(6)]
    st = built_lib.pb_quantize_dual(x.data_ptr(), 1, 1, 128, 512, 0, *[o.data_ptr() for o in outs], outs[0].data_ptr(), 1 << 16, None)
    assert st == _lib.PB_ERR_UNSUPPORTED


@pytest.mark.parametrize("rows,cols", [(128, 1024), (200, 4096), (1000, 2048)])
def test_relu2_requantize_has_the_bits_of_the_three_steps(built_lib, rows, cols):
    from pratchya_b200._qualia import fake_quantize_impl
    y = synth((rows, cols), seed=rows + cols, outliers=0.01)
    y.reshape(-1)[:1024] = 0.0
    y.reshape(-1)[1024:2048] = -np.abs(y.reshape(-1)[1024:2048])          # a super-group that relu wipes out
    yt = to_torch(y)
    k = torch.relu(fake_quantize_impl(yt, (1, 128), torch.float32)) ** 2
    want = quantize_impl(k, (1, 128))
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device="cuda")
    sc8 = torch.empty_like(want[1])
    sc32 = torch.empty_like(want[2])
    _lib.check(built_lib.pb_relu2_requantize(yt.data_ptr(), rows, cols, 0, q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(),
                                             None, None, 0, torch.cuda.current_stream().cuda_stream))
    assert_triple_equal(np_triple((q, sc8, sc32)), np_triple(want), "fused middle vs fake-quantize, relu^2, quantize")
    # and against the oracle's three steps
    oq = oracle.quantize_impl(np.asarray(y), (1, 128))
    kk = np.maximum(oracle.dequantize_impl(*oq, np.float32, (1, 128)), 0).astype(np.float32) ** 2
    ok = oracle.quantize_impl(kk.astype(np.float32), (1, 128))
    assert_triple_equal(np_triple((q, sc8, sc32)), (ok[0].view(np.uint8), ok[1].view(np.uint8), ok[2]), "fused middle vs oracle")
    st = built_lib.pb_relu2_requantize(yt.data_ptr(), rows, 512, 0, q.data_ptr(), sc8.data_ptr(), sc32.data_ptr(), None, None, 0, None)
    assert st == _lib.PB_ERR_UNSUPPORTED


def test_channel_mix_ffn_fused_equals_literal(built_lib):
    from pratchya_b200._nnx_impl import ChannelMixFFN
    ffn = ChannelMixFFN(1024, 4096, generator=torch.Generator(device="cuda").manual_seed(21))
    for x in (to_torch(synth((2, 96, 1024), seed=5)), to_torch(synth((256, 1024), seed=6))):
        got = ffn(x)
        assert ffn.w_k._steps and ffn.w_v._steps and all(v is not None for v in ffn.w_v._steps.values())
        want = ffn.literal(x)
        assert got.shape == want.shape and got.dtype == want.dtype
        assert torch.equal(got, want)
    xb = to_torch(synth((256, 1024), seed=7).astype(BF16))          # bf16 input: the literal sequence
    assert torch.equal(ffn(xb), ffn.literal(xb))


def test_step_captures_into_a_cuda_graph(built_lib):
    """The calls are stream-ordered and allocate nothing, so a quantize + GEMM step records into a CUDA
    graph as it is; replaying the graph on new input gives the bits of the eager calls."""
    m, n, k = 512, 1024, 2048
    wq, w_t = weight(k, n, seed=8)
    x = to_torch(synth((m, k), seed=1).astype(BF16))
    q = torch.empty((m, k), dtype=torch.uint8, device="cuda")
    s8 = torch.empty(m * k // 128, dtype=torch.uint8, device="cuda")
    s32 = torch.empty(m * k // 1024, dtype=torch.float32, device="cuda")
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    a = _lib.Operand(q.data_ptr(), s8.data_ptr(), s32.data_ptr(), m, k, 1, 128, 0, 0)
    b = _ops._operand(w_t, wq[1], wq[2], n, k, (128, 128), 1)
    ws_bytes = built_lib.pb_gemm_workspace_size(a, b)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")

    def step(stream, flags):
        _lib.check(built_lib.pb_quantize_for_gemm(x.data_ptr(), 1, m, k, 0, q.data_ptr(), s8.data_ptr(), s32.data_ptr(), b, ws.data_ptr(), ws_bytes, stream))
        _lib.check(built_lib.pb_gemm_tn_ex(a, b, y.data_ptr(), 1, n, ws.data_ptr(), ws_bytes, flags, stream))

    step(torch.cuda.current_stream().cuda_stream, _ops.GEMM_A_PREPARED)          # also prepares the weight's scales
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            step(side.cuda_stream, _ops.GEMM_A_PREPARED | _ops.GEMM_B_PREPARED)
    torch.cuda.current_stream().wait_stream(side)
    x.copy_(to_torch(synth((m, k), seed=2, scale=7.0).astype(BF16)))             # new input in the same buffer
    y.zero_()
    graph.replay()
    torch.cuda.synchronize()
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    want = matmul_impl(*quantize_impl(x, (1, 128)), *wq, (1, 128), (128, 128), y_fp8_t=w_t, out_dtype=torch.bfloat16)
    assert torch.equal(y, want)
