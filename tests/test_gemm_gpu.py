"""GPU parity of the block-scaled FP8 matmul with the oracle's dq(A) @ dq(B) on the same
quantized operands.  Tolerance: max |got - ref| <= 1e-2 * max |ref| per output matrix, and
<= 1e-2 relative on entries with |ref| above 5% of the matrix maximum (the tensor core sums
exact fp8 products in fp32; the bound covers its accumulation order)."""
import numpy as np
import pytest
import torch

from helpers import BF16, bytes_of, check_close, from_torch, oracle, synth, to_torch
from pratchya_b200 import _lib
from pratchya_b200._qualia import matmul_impl, quantize_impl, quantize_transposed_impl
from pratchya_b200._qualia import _ops

pytestmark = pytest.mark.gpu

def gpu_triple(x, grid):
    return quantize_impl(to_torch(x), grid)


def np_triple(t):
    q, s8, s32 = t
    return (bytes_of(q).view(oracle.E4M3), bytes_of(s8), from_torch(s32))


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 128, 512), (128, 256, 1024), (256, 256, 2048),
                                   (200, 384, 1024), (1024, 1024, 2048), (384, 128, 2304), (128, 1280, 4096)])
def test_forward_matmul_matches_oracle(built_lib, m, n, k):
    x = synth((m, k), seed=m + n + k, outliers=0.01)
    w = synth((k, n), seed=m * 7 + n, scale=0.02, outliers=0)
    xq, wq = gpu_triple(x, (1, 128)), gpu_triple(w, (128, 128))
    if oracle.group_geometry(m, k, (1, 128))[1] != 8:
        pytest.skip("activation super-group is not 8 blocks: falls back to the literal path")
    got = matmul_impl(*xq, *wq, (1, 128), (128, 128))
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 128), (128, 128), acc=np.float64)
    check_close(got.cpu().numpy(), ref, f"fwd {m}x{n}x{k}")


def test_bf16_output_and_student_t(built_lib):
    m, n, k = 512, 512, 2048
    x = synth((m, k), seed=1, dist="student_t", outliers=0).astype(BF16)
    w = synth((k, n), seed=2, scale=0.02, outliers=0).astype(BF16)
    xq, wq = gpu_triple(x, (1, 128)), gpu_triple(w, (128, 128))
    got = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 128), (128, 128), acc=np.float64)
    check_close(from_torch(got).astype(np.float32), ref, "bf16 out")


def test_dgrad_and_wgrad_operand_forms(built_lib):
    """dgrad: A = Q(g,(1,128)) [M,N], B = the weight as stored [K,N] (N is the depth).
    wgrad: A = Q(x^T,(1,128)) [K,M], B = Q(g^T,(1,128)) [N,M] (tokens are the depth)."""
    m, n, k = 1024, 512, 256
    x = synth((m, k), seed=3)
    w = synth((k, n), seed=4, scale=0.02, outliers=0)
    g = synth((m, n), seed=5, scale=1e-3, outliers=0)
    wq = gpu_triple(w, (128, 128))
    gq = gpu_triple(g, (1, 128))
    a = _ops._operand(gq[0], gq[1], gq[2], m, n, (1, 128))
    b = _ops._operand(wq[0], wq[1], wq[2], k, n, (128, 128))
    dx = _ops.gemm_tn(a, b, torch.float32, gq[0].device)
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    g_hat = oracle.dequantize_impl(*np_triple(gq), np.float64, (1, 128))
    w_hat = oracle.dequantize_impl(*np_triple(wq), np.float64, (128, 128))
    check_close(dx.cpu().numpy(), g_hat @ w_hat.T, "dgrad")

    xt = quantize_transposed_impl(to_torch(x), 128)
    gt = quantize_transposed_impl(to_torch(g), 128)
    want_xt = oracle.quantize_impl(np.ascontiguousarray(x.T), (1, 128))
    assert np.array_equal(bytes_of(xt[0]), bytes_of(want_xt[0])) and np.array_equal(bytes_of(xt[1]), want_xt[1])
    assert np.array_equal(from_torch(xt[2]), want_xt[2])
    a = _ops._operand(xt[0], xt[1], xt[2], k, m, (1, 128))
    b = _ops._operand(gt[0], gt[1], gt[2], n, m, (1, 128))
    dw = _ops.gemm_tn(a, b, torch.float32, xt[0].device)
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    xt_hat = oracle.dequantize_impl(*np_triple(xt), np.float64, (1, 128))
    gt_hat = oracle.dequantize_impl(*np_triple(gt), np.float64, (1, 128))
    check_close(dw.cpu().numpy(), xt_hat @ gt_hat.T, "wgrad")


def test_slab_supergroups_of_a_large_weight(built_lib):
    """A weight with more than 1024 blocks has several fp32 amax slabs along the depth."""
    m, n, k = 128, 4096, 8192          # 64 x 32 blocks -> K = 1024 blocks = 32 block rows per slab
    x = synth((m, k), seed=6)
    w = synth((k, n), seed=7, scale=0.02, outliers=0)
    w[:4096] *= 8.0                     # make the two slabs differ
    xq, wq = gpu_triple(x, (1, 128)), gpu_triple(w, (128, 128))
    assert wq[2].numel() == 2
    got = matmul_impl(*xq, *wq, (1, 128), (128, 128))
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 128), (128, 128), acc=np.float64)
    check_close(got.cpu().numpy(), ref, "slabs")


def test_literal_path_for_small_grids(built_lib):
    x = synth((64, 96), seed=8)
    w = synth((96, 48), seed=9, scale=0.02, outliers=0)
    xq, wq = gpu_triple(x, (1, 16)), gpu_triple(w, (16, 16))
    got = matmul_impl(*xq, *wq, (1, 16), (16, 16))
    ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 16), (16, 16), acc=np.float64)
    check_close(got.cpu().numpy(), ref, "literal")


def test_transposed_quantizer_bit_exact(built_lib):
    for shape, dt in [((1024, 256), np.float32), ((2048, 192), BF16), ((1024, 100), np.float32), ((128, 64), BF16)]:
        x = synth(shape, seed=10, outliers=0.01).astype(dt)
        got = quantize_transposed_impl(to_torch(x), 128)
        want = oracle.quantize_impl(np.ascontiguousarray(x.T), (1, 128))
        assert np.array_equal(bytes_of(got[0]), bytes_of(want[0])), shape
        assert np.array_equal(bytes_of(got[1]), want[1]) and np.array_equal(from_torch(got[2]), want[2])


@pytest.mark.parametrize("m,n,k", [(512, 512, 4096), (2048, 2048, 8192), (300, 700, 5120)])
def test_few_tiles_split_over_k(built_lib, m, n, k):
    """f32 outputs with few tiles and a long K run as two half-K work units per tile that add into a
    zeroed D: same tolerance against the oracle, bit-identical from run to run, and equal within
    rounding of the output type to the bf16 result (which is never split)."""
    if n % 128:
        n = (n // 128 + 1) * 128
    x = synth((m, k), seed=m + k, outliers=0.01)
    w = synth((k, n), seed=n, scale=0.02, outliers=0)
    xq, wq = gpu_triple(x, (1, 128)), gpu_triple(w, (128, 128))
    if oracle.group_geometry(m, k, (1, 128))[1] != 8:
        pytest.skip("activation super-group is not 8 blocks")
    got = matmul_impl(*xq, *wq, (1, 128), (128, 128))
    again = matmul_impl(*xq, *wq, (1, 128), (128, 128))
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    assert torch.equal(got, again)
    ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 128), (128, 128), acc=np.float64)
    check_close(got.cpu().numpy(), ref, f"split {m}x{n}x{k}")
    as_bf16 = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
    scale = float(np.abs(ref).max())
    assert (got - as_bf16.float()).abs().max().item() <= 2.0 ** -7 * scale


def test_random_shapes_against_f64_product(built_lib):
    """Seeded sweep over row counts, widths and depths that exercise partial tiles, both kernels (operands of
    at most 128 rows use the single-CTA one), bands, the split over K and both output types; the check is
    the f64 product of the dequantized operands (the dequantizer itself is bit-exact against the oracle)."""
    import random
    from pratchya_b200._qualia import dequantize_impl
    rnd = random.Random(7)
    done = 0
    while done < 14:
        m = rnd.choice([8, 64, 128, 136, 264, 520, 1024, 2048, 4096])
        n = 128 * rnd.choice([1, 2, 3, 5, 8, 17, 32, 64])
        k = 128 * rnd.choice([1, 2, 4, 8, 16, 24, 32, 64])
        if (m * k // 128) % 8:
            continue
        done += 1
        out = rnd.choice([torch.float32, torch.bfloat16])
        x = torch.randn(m, k, device="cuda", generator=torch.Generator(device="cuda").manual_seed(done)) * rnd.choice([1e-3, 1.0, 30.0])
        w = torch.randn(k, n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 + done)) * 0.02
        xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
        got = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=out)
        _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
        ref = dequantize_impl(*xq, torch.float32, (1, 128)).double() @ dequantize_impl(*wq, torch.float32, (128, 128)).double()
        scale = ref.abs().max().item()
        err = (got.double() - ref).abs().max().item()
        tol = 1e-5 if out == torch.float32 else 2.0 ** -7
        assert err <= tol * scale, f"{m}x{n}x{k} {out}: max abs err {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("grid", [(128, 128), (128, 1)])
@pytest.mark.parametrize("m,k,n", [(32768, 128, 2048), (16384, 256, 2048), (32768, 128, 256), (8192, 384, 1024), (64, 128, 65536)])
def test_shallow_products_with_many_tiles_per_cta(built_lib, m, k, n, grid):
    """One to three k-blocks per tile and many tiles per CTA (the reference's LoRA up projection at 8 x 4096 tokens:
    rank 128 -> 2048 channels): every pipeline step then brings new scale factors, so their shared-memory slots and
    TMEM sets turn over at the pipeline's own pace.  Checked against the f64 product of the dequantized operands
    and for equal bits from run to run."""
    from pratchya_b200._qualia import dequantize_impl
    gen = torch.Generator(device="cuda").manual_seed(m + k + n)
    x = torch.tanh(torch.randn(m, k, device="cuda", generator=gen) * 2.0)
    x[::7] *= 1e-3                                                # rows of very different scale: a stale scale factor shows
    w = torch.randn(k, n, device="cuda", generator=gen) * 0.1
    w[:, ::5] *= 40.0
    xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, grid)
    ref = dequantize_impl(*xq, torch.float32, (1, 128)).double() @ dequantize_impl(*wq, torch.float32, grid).double()
    scale = ref.abs().max().item()
    first = None
    for _ in range(4):
        got = matmul_impl(*xq, *wq, (1, 128), grid)
        _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
        err = (got.double() - ref).abs().max().item()
        assert err <= 1e-5 * scale, f"{m}x{n}x{k} on {grid}: max abs err {err:.3e} against a largest magnitude of {scale:.3e}"
        first = got if first is None else first
        assert torch.equal(got, first)


@pytest.mark.parametrize("m,k,n", [(32768, 2048, 128), (4096, 2048, 65536), (8192, 768, 2048)])
def test_column_scaled_weights_at_the_model_sizes(built_lib, m, k, n):
    """(128,1) weights at the sizes the end-to-end model uses them: a LoRA down projection over 8 x 4096 tokens, the
    lm_head's 65536 columns, and a depth that is not a multiple of four k-blocks.  Their chunks are single k-blocks
    (the epilogue form with one fp32 factor per eight columns, fetched a chunk ahead); many tiles per CTA."""
    from pratchya_b200._qualia import dequantize_impl
    gen = torch.Generator(device="cuda").manual_seed(m + k + n)
    x = torch.randn(m, k, device="cuda", generator=gen)
    x[::5] *= 1e-2
    w = torch.randn(k, n, device="cuda", generator=gen) * 0.05
    w[:, ::9] *= 30.0                                            # neighbouring column groups with very different factors
    xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 1))
    assert _ops._tensor_core_eligible(xq[0], wq[0], (1, 128), (128, 1))
    got = matmul_impl(*xq, *wq, (1, 128), (128, 1))
    again = matmul_impl(*xq, *wq, (1, 128), (128, 1))
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    assert torch.equal(got, again)
    w_hat = dequantize_impl(*wq, torch.float32, (128, 1)).double()
    x_hat = dequantize_impl(*xq, torch.float32, (1, 128))
    worst, scale = 0.0, 0.0
    for r0 in range(0, m, 4096):                                 # the f64 product in row bands
        ref = x_hat[r0:r0 + 4096].double() @ w_hat
        worst = max(worst, (got[r0:r0 + 4096].double() - ref).abs().max().item())
        scale = max(scale, ref.abs().max().item())
    assert worst <= 1e-5 * scale, f"{m}x{n}x{k}: max abs err {worst:.3e} against a largest magnitude of {scale:.3e}"


@pytest.mark.parametrize("m,k,n", [(256, 2048, 64), (512, 128, 2048), (384, 1024, 4096), (128, 2048, 48)])
def test_column_scaled_weights_run_on_the_tensor_cores(built_lib, m, k, n):
    """Weights on the (128,1) grid -- the reference's LoRA down/up, gate and lm_head kernels
    (pratchya/_nnx_impl/_module.py:82-84, 326; _model.py:77): one e8m0 byte per column and 128-deep block, an
    fp32 amax per eight adjacent columns of a 128-row band.  Same check as the (128,128) weights: the oracle's
    f64 product of the same quantized operands."""
    x = synth((m, k), seed=m + k, outliers=0.01)
    w = synth((k, n), seed=n, scale=0.05, outliers=0.02)          # outliers make neighbouring column groups differ
    xq, wq = gpu_triple(x, (1, 128)), gpu_triple(w, (128, 1))
    assert _ops._tensor_core_eligible(xq[0], wq[0], (1, 128), (128, 1))
    for out in (torch.float32, torch.bfloat16):
        got = matmul_impl(*xq, *wq, (1, 128), (128, 1), out_dtype=out)
        _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
        ref = oracle.matmul_impl(*np_triple(xq), *np_triple(wq), (1, 128), (128, 1), acc=np.float64)
        err = check_close(got.float().cpu().numpy(), ref, f"(128,1) weight {m}x{n}x{k} {out}")
    # the literal route (dequantize both, f32 library matmul) agrees with it
    lit = _ops._matmul_f32(_ops.dequantize_impl(*xq, torch.float32, (1, 128)), _ops.dequantize_impl(*wq, torch.float32, (128, 1)))
    assert (lit - matmul_impl(*xq, *wq, (1, 128), (128, 1))).abs().max().item() <= 1e-4 * np.abs(ref).max()


def test_low_rank_ffn_matches_the_oracle_chain(built_lib):
    """LowRankFFN (pratchya/_nnx_impl/_module.py:74-89): up(tanh(down(x))) with both kernels on (blk,1) grids, each
    Linear returning dq(q(product, (1,1))) -- on the (1,1) grid every element is its own block, so the fake
    quantization is exact up to the f32 -> bf16 -> fp8 cast of +-128 and a scale of |y|: the layer's value is
    the plain product to f32 rounding.  Checked against the oracle's chain on the layer's own quantized kernels."""
    from pratchya_b200._nnx_impl import LowRankFFN
    hidden, rank, rows = 1024, 128, 256
    gen = torch.Generator(device="cuda").manual_seed(3)
    layer = LowRankFFN(hidden, rank, (128, 128), generator=gen)
    assert layer.down.kernel.tgrid == (128, 1) and layer.up.kernel.tgrid == (128, 1)
    x = synth((rows, hidden), seed=5, outliers=0.01)
    got = layer(to_torch(x)).cpu().numpy()
    kd, ku = layer.down.kernel, layer.up.kernel
    down = oracle.linear_forward(x, np_triple((kd.get_value(), kd.sc_fp8, kd.sc_fp32)), (128, 1))
    want = oracle.linear_forward(np.tanh(down).astype(np.float32), np_triple((ku.get_value(), ku.sc_fp8, ku.sc_fp32)), (128, 1))
    assert got.shape == want.shape == (rows, hidden)
    scale = np.abs(want).max()
    # tanh differs in the last bit between numpy and the device, which can move an element of the second
    # quantization across an fp8 rounding boundary: 5e-3 of the maximum leaves room for a few of those
    assert np.abs(got - want).max() <= 5e-3 * scale, f"LowRankFFN differs from the oracle chain by {np.abs(got - want).max() / scale:.2e} of its maximum"
