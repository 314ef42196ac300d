"""GPU parity on the shapes the benchmark configurations name, at full size.

The quantizers are compared bit for bit with the oracle on seeded 1024-row bands of the full input
(a (1,128) row band, and a 1024-token band of the transposed form, reproduce the bytes and scales of
the full tensor: super-groups never cross them).  The matmuls run at full size and are compared with
the oracle's f64 product of the same quantized operands on a seeded subset of output rows (all
columns) -- tolerance as in test_gemm_gpu.py: 1e-2 of the matrix maximum and 1e-2 relative on large
entries; the observed error is printed."""
import numpy as np
import pytest
import torch

from helpers import bytes_of, check_close, from_torch, oracle
from pratchya_b200 import _lib
from pratchya_b200._qualia import _ops, matmul_impl, quantize_impl, quantize_transposed_impl

pytestmark = pytest.mark.gpu

E4M3, E5M2 = oracle.E4M3, oracle.E5M2


def seeded(shape, seed, scale=1.0, dist="normal", dtype=torch.bfloat16):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    if dist == "student_t":          # t(3) = z / sqrt(chi2_3 / 3), built from seeded normals
        z = torch.randn(shape, device="cuda", generator=gen)
        chi = sum(torch.randn(shape, device="cuda", generator=gen) ** 2 for _ in range(3)) / 3.0
        x = z / chi.sqrt()
    else:
        x = torch.randn(shape, device="cuda", generator=gen)
    return (x * scale).to(dtype)


def to_np(t):
    return from_torch(t.contiguous())


def np_dtype(q):
    return E5M2 if q.dtype == torch.float8_e5m2 else E4M3


def rows_of_row128(triple, idx, cols):
    """The triple of the rows `idx` of a (1,128)-quantized [rows, cols] array (cols % 1024 == 0)."""
    q, s8, s32 = triple
    rows = q.shape[0]
    gpr = cols // 1024
    i = torch.as_tensor(idx, device=q.device)
    qs = bytes_of(q.view(torch.uint8)[i]).view(np_dtype(q))
    s8s = bytes_of(s8.view(torch.uint8).view(rows, gpr, 8)[i].reshape(-1, 8))
    s32s = from_torch(s32.view(rows, gpr)[i].reshape(-1, 1, 1))
    return qs, s8s, s32s


def full_np(triple):
    q, s8, s32 = triple
    return bytes_of(q).view(np_dtype(q)), bytes_of(s8), from_torch(s32)


def assert_band_bits(got, x, r0, r1, grid=(1, 128), fmt="e4m3"):
    """Rows [r0, r1) of a (1,128)-quantized array against the oracle run on that band alone."""
    q, s8, s32 = got
    cols = x.shape[1]
    want = oracle.quantize_impl(to_np(x[r0:r1]), grid, fmt)
    gpr = cols // 1024
    assert np.array_equal(bytes_of(q[r0:r1]), bytes_of(want[0])), f"fp8 bytes differ in rows {r0}:{r1}"
    assert np.array_equal(bytes_of(s8.view(torch.uint8)[r0 * gpr:r1 * gpr]), want[1]), f"e8m0 bytes differ in rows {r0}:{r1}"
    assert np.array_equal(from_torch(s32[r0 * gpr:r1 * gpr]).view(np.uint32), want[2].view(np.uint32)), f"fp32 scales differ in rows {r0}:{r1}"


def assert_token_band_bits(got_t, x, r0, fmt="e4m3"):
    """Tokens [r0, r0+1024) of quantize_impl(x^T, (1,128)) against the oracle run on that band's transpose."""
    qt, s8, s32 = got_t
    rows, cols = x.shape
    want = oracle.quantize_impl(np.ascontiguousarray(to_np(x[r0:r0 + 1024]).T), (1, 128), fmt)
    g = r0 // 1024
    assert np.array_equal(bytes_of(qt[:, r0:r0 + 1024]), bytes_of(want[0])), f"transposed fp8 bytes differ in tokens {r0}:{r0 + 1024}"
    assert np.array_equal(bytes_of(s8.view(torch.uint8).view(cols, rows // 1024, 8)[:, g]), want[1])
    assert np.array_equal(from_torch(s32.view(cols, rows // 1024)[:, g]).view(np.uint32), want[2].reshape(-1).view(np.uint32))


def check_gemm_rows(built_lib, d, a_triple, a_cols, b_hat64, idx, what):
    """d[idx, :] against dq(A)[idx, :] @ b_hat64 in f64."""
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    a_hat = oracle.dequantize_impl(*rows_of_row128(a_triple, idx, a_cols), np.float64, (1, 128))
    ref = a_hat @ b_hat64
    got = d[torch.as_tensor(idx, device=d.device)].float().cpu().numpy()
    err = check_close(got, ref, what)
    print(f"{what}: max error {err:.2e} of the matrix maximum on {len(idx)} rows")


def subset(n, count, seed):
    return np.sort(np.random.default_rng(seed).choice(n, size=count, replace=False))


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_config2_forward_at_full_size(built_lib, out_dtype):
    """configs[1]: X bf16 [8192,2048] ~ N(0,1) on (1,128), W bf16 [2048,8192] ~ N(0,0.02) on (128,128)."""
    m, k, n = 8192, 2048, 8192
    x, w = seeded((m, k), 21), seeded((k, n), 22, scale=0.02)
    xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
    want_w = oracle.quantize_impl(to_np(w), (128, 128))
    assert np.array_equal(bytes_of(wq[0]), bytes_of(want_w[0])) and np.array_equal(bytes_of(wq[1]), want_w[1])
    assert np.array_equal(from_torch(wq[2]), want_w[2])
    for r0 in (0, 3072, 7168):
        assert_band_bits(xq, x, r0, r0 + 1024)
    y = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=out_dtype)
    w_hat = oracle.dequantize_impl(*want_w, np.float64, (128, 128))
    check_gemm_rows(built_lib, y, xq, k, w_hat, subset(m, 512, 1), f"config 2 forward, {out_dtype}")


def test_config3_quantizers_at_full_size(built_lib):
    """configs[2]: X [32768,2048] and dY [32768,8192] ~ N(0,1e-3), row form and token (transposed) form,
    dY in the reference's e4m3 and in the e5m2 extension."""
    m = 32768
    x = seeded((m, 2048), 31)
    xq = quantize_impl(x, (1, 128))
    xt = quantize_transposed_impl(x, 128)
    for r0 in (0, 13312, 31744):
        assert_band_bits(xq, x, r0, r0 + 1024)
        assert_token_band_bits(xt, x, r0)
    del xq, xt
    dy = seeded((m, 8192), 32, scale=1e-3)
    for fmt in ("e4m3", "e5m2"):
        gq = quantize_impl(dy, (1, 128), out_format=fmt)
        gt = quantize_transposed_impl(dy, 128, out_format=fmt)
        for r0 in (1024, 30720):
            assert_band_bits(gq, dy, r0, r0 + 1024, fmt=fmt)
            assert_token_band_bits(gt, dy, r0, fmt=fmt)
        del gq, gt
    # both forms from one call
    (q1, s1, t1), (q2, s2, t2) = _ops.quantize_dual_impl(x)
    assert_band_bits((q1, s1, t1), x, 5120, 6144)
    assert_token_band_bits((q2, s2, t2), x, 5120)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape,fmt", [((4096, 4096), "e4m3"), ((3, 2048, 2048), "e5m2"), ((1024, 16384), "e4m3")])
def test_persistent_transposed_quantizer_against_the_full_oracle(built_lib, shape, fmt, dtype):
    """Shapes with enough 1024-row x 64-byte tiles (32 bf16 or 16 f32 columns) to run the persistent TMA-staged form of
    the single-pass transposed quantizer, compared with the oracle over the whole array (not bands), twice in a row
    (the second call reuses the kernel's barriers and buffers from a fresh launch)."""
    x = seeded(shape, 61, scale=3.0, dtype=dtype)
    x.view(-1)[::4097] *= 64.0                      # outliers
    x[..., :1024, 5] = 0.0                         # an all-zero super-group
    xn = to_np(x)
    lead = shape[:-2]
    for _ in range(2):
        got = quantize_transposed_impl(x, 128, out_format=fmt)
        torch.cuda.synchronize()
        _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
        for idx in np.ndindex(*lead) if lead else [()]:
            want = oracle.quantize_impl(np.ascontiguousarray(xn[idx].T), (1, 128), fmt)
            assert np.array_equal(bytes_of(got[0][idx]), bytes_of(want[0])), f"fp8 bytes differ in slice {idx}"
            assert np.array_equal(bytes_of(got[1][idx]), want[1]), f"e8m0 bytes differ in slice {idx}"
            assert np.array_equal(from_torch(got[2][idx]).view(np.uint32), want[2].view(np.uint32)), f"fp32 scales differ in slice {idx}"


@pytest.mark.parametrize("k_in,n_out", [(2048, 2048), (2048, 8192), (8192, 2048)])
@pytest.mark.parametrize("grad_format", ["e4m3", "e5m2"])
def test_config3_triple_at_full_size(built_lib, k_in, n_out, grad_format):
    """forward, dgrad and wgrad of one projection at M = 32768 tokens against the oracle on the same
    quantized operands; dY is e4m3 (the reference's dtype) or e5m2 (the extension config 3 names)."""
    m = 32768
    x, w = seeded((m, k_in), 41), seeded((k_in, n_out), 42, scale=0.02)
    dy = seeded((m, n_out), 43, scale=1e-3)
    dev = x.device
    op = _ops._operand
    wq = quantize_impl(w, (128, 128))
    w_hat = oracle.dequantize_impl(*full_np(wq), np.float64, (128, 128))
    if grad_format == "e4m3":          # the forward does not depend on the gradient's format: once is enough
        xq = quantize_impl(x, (1, 128))
        y = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
        check_gemm_rows(built_lib, y, xq, k_in, w_hat, subset(m, 256, 2), f"fwd {k_in}->{n_out}")
        del xq, y
    gq = quantize_impl(dy, (1, 128), out_format=grad_format)
    dx = _ops.gemm_tn(op(gq[0], gq[1], gq[2], m, n_out, (1, 128)), op(wq[0], wq[1], wq[2], k_in, n_out, (128, 128)), torch.bfloat16, dev)
    check_gemm_rows(built_lib, dx, gq, n_out, w_hat.T, subset(m, 256, 3), f"dgrad {k_in}->{n_out} dY {grad_format}")
    del gq, dx
    xt = quantize_transposed_impl(x, 128)
    gt = quantize_transposed_impl(dy, 128, out_format=grad_format)
    dw = _ops.gemm_tn(op(xt[0], xt[1], xt[2], k_in, m, (1, 128)), op(gt[0], gt[1], gt[2], n_out, m, (1, 128)), torch.float32, dev)
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    ri, ci = subset(k_in, 48, 4), subset(n_out, 384, 5)
    xt_hat = oracle.dequantize_impl(*rows_of_row128(xt, ri, m), np.float64, (1, 128))
    gt_hat = oracle.dequantize_impl(*rows_of_row128(gt, ci, m), np.float64, (1, 128))
    got = dw[torch.as_tensor(ri, device=dev)][:, torch.as_tensor(ci, device=dev)].cpu().numpy()
    err = check_close(got, xt_hat @ gt_hat.T, f"wgrad {k_in}->{n_out} dY {grad_format}")
    print(f"wgrad {k_in}->{n_out} dY {grad_format}: max error {err:.2e} of the matrix maximum")


def test_config4_shard_student_t_and_slab_weight(built_lib):
    """configs[3]: one GPU's 8192-row shard of Student-t(3) activations at d_model 4096 against the
    [4096,16384] up-projection, whose (128,128) scales fall into four fp32 slabs."""
    m, k, n = 8192, 4096, 16384
    x, w = seeded((m, k), 51, dist="student_t"), seeded((k, n), 52, scale=0.02)
    xq, wq = quantize_impl(x, (1, 128)), quantize_impl(w, (128, 128))
    assert wq[2].numel() == 4
    want_x = oracle.quantize_impl(to_np(x), (1, 128))
    assert np.array_equal(bytes_of(xq[0]), bytes_of(want_x[0])) and np.array_equal(bytes_of(xq[1]), want_x[1])
    assert np.array_equal(from_torch(xq[2]).view(np.uint32), want_x[2].view(np.uint32))
    want_w = oracle.quantize_impl(to_np(w), (128, 128))
    assert np.array_equal(bytes_of(wq[0]), bytes_of(want_w[0])) and np.array_equal(bytes_of(wq[1]), want_w[1])
    assert np.array_equal(from_torch(wq[2]), want_w[2])
    y = matmul_impl(*xq, *wq, (1, 128), (128, 128), out_dtype=torch.bfloat16)
    w_hat = oracle.dequantize_impl(*want_w, np.float64, (128, 128))
    check_gemm_rows(built_lib, y, xq, k, w_hat, subset(m, 192, 6), "config 4 forward shard")
    # the shard reproduces the rows of a larger activation: quantize two shards as one tensor
    big = torch.cat([x, seeded((m, k), 53, dist="student_t")])
    bq = quantize_impl(big, (1, 128))
    assert torch.equal(bq[0][:m].view(torch.uint8), xq[0].view(torch.uint8))
    assert torch.equal(bq[1].view(torch.uint8)[: m * k // 1024], xq[1].view(torch.uint8))
    # dgrad against the same weight: its bytes as stored, slabs along the depth
    dy = seeded((m, n), 54, scale=1e-3)
    gq = quantize_impl(dy, (1, 128))
    op = _ops._operand
    dx = _ops.gemm_tn(op(gq[0], gq[1], gq[2], m, n, (1, 128)), op(wq[0], wq[1], wq[2], k, n, (128, 128)), torch.bfloat16, x.device)
    check_gemm_rows(built_lib, dx, gq, n, w_hat.T, subset(m, 128, 7), "config 4 dgrad shard")
