"""Shared helpers of the parity tests (test infrastructure; may use oracle/)."""
import ml_dtypes
import numpy as np

from oracle import qarr_oracle as oracle

BF16 = ml_dtypes.bfloat16


def synth(shape, seed, dist="normal", outliers=0.01, scale=1.0, dtype=np.float32):
    """Seeded synthetic tensors with the value distributions of the benchmark configs:
    N(0, scale^2) with a seeded fraction of entries multiplied by 64, or Student-t(3)."""
    rng = np.random.default_rng(seed)
    if dist == "student_t":
        x = rng.standard_t(3, size=shape).astype(np.float32) * np.float32(scale)
    else:
        x = rng.standard_normal(shape).astype(np.float32) * np.float32(scale)
    if outliers:
        mask = rng.random(shape) < outliers
        x = np.where(mask, x * np.float32(64.0), x).astype(np.float32)
    return x.astype(dtype)


def to_torch(x, device="cuda"):
    import torch
    if x.dtype == BF16:
        return torch.from_numpy(x.view(np.uint16).copy()).view(torch.bfloat16).to(device)
    return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def bytes_of(t):
    """uint8 numpy view of a torch fp8/e8m0 tensor or an ml_dtypes array."""
    import torch
    if isinstance(t, torch.Tensor):
        return t.contiguous().reshape(-1).view(torch.uint8).cpu().numpy().reshape(tuple(t.shape))
    return np.ascontiguousarray(t).reshape(-1).view(np.uint8).reshape(np.shape(t))


def from_torch(t):
    import torch
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).cpu().numpy().view(BF16)
    return t.cpu().numpy()


def assert_triple_equal(got, want, what=""):
    gq, g8, g32 = got
    wq, w8, w32 = want
    gq, wq = bytes_of(gq), bytes_of(wq)
    assert gq.shape == wq.shape, f"{what}: value shape {gq.shape} vs {wq.shape}"
    bad = np.flatnonzero(gq.reshape(-1) != wq.reshape(-1))
    assert bad.size == 0, f"{what}: {bad.size} fp8 bytes differ, first at {bad[:5]}: got {gq.reshape(-1)[bad[:5]]} want {wq.reshape(-1)[bad[:5]]}"
    g8, w8 = bytes_of(g8), bytes_of(w8)
    assert g8.shape == w8.shape, f"{what}: sc8 shape {g8.shape} vs {w8.shape}"
    assert np.array_equal(g8, w8), f"{what}: e8m0 bytes differ"
    g32 = from_torch(g32) if not isinstance(g32, np.ndarray) else g32
    assert g32.shape == w32.shape, f"{what}: sc32 shape {g32.shape} vs {w32.shape}"
    assert np.array_equal(g32.view(np.uint32), w32.view(np.uint32)), f"{what}: fp32 scales differ"


REL_TOL = 1e-2


def check_close(got, ref, what):
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    scale = np.abs(ref).max()
    err = np.abs(got - ref)
    assert err.max() <= REL_TOL * scale, f"{what}: max abs err {err.max():.3e} vs scale {scale:.3e}"
    big = np.abs(ref) > 0.05 * scale
    if big.any():
        rel = (err[big] / np.abs(ref[big])).max()
        assert rel <= REL_TOL, f"{what}: max rel err {rel:.3e}"
    return err.max() / scale


def assert_fake_quantized_close(got, want, what, boundary_fraction=0.01, bf16=False):
    """Two arrays that are both the fp8 (fake-)quantization of almost the same f32 matrix (their sources agree to
    ~1e-6): equal to 1e-5 (one bf16 ulp if `bf16`) on all but `boundary_fraction` of the elements -- those whose
    source sits on a rounding boundary of the cast -- and within one fp8 step of each other everywhere
    (2^-3 of the value; 2^-6 of the array's maximum covers the small values of a block with a large scale)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    scale = np.abs(want).max()
    diff = np.abs(got - want)
    eps = 2.0 ** -7 if bf16 else 1e-5
    off = diff > eps * np.abs(want) + 1e-9 * scale
    assert off.mean() <= boundary_fraction, f"{what}: {off.mean():.4f} of the elements differ (allowed {boundary_fraction})"
    worst = (diff - 2.0 ** -3 * np.abs(want)).max()
    assert worst <= 2.0 ** -6 * scale, f"{what}: a difference exceeds one fp8 step by {worst / scale:.2e} of the maximum"
