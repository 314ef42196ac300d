"""GPU parity of the WKV-7 state scan kernel with the oracle's restatement of
pratchya/_nnx_impl/_module.py:187-207.  Floating point: the kernel sums in fp32 in its own order (the
reference's own order is whatever XLA gives its batched matmuls), so the check is against the oracle
run in float64, with the tolerance 2e-5 of the largest |out| (and of the largest |state|) for sequences
up to 4096 steps; the oracle's own float32 run is held to the same bound, which shows the bound is
the precision of the recurrence, not slack for the kernel."""
import numpy as np
import pytest
import torch

from oracle import wkv7_oracle
from pratchya_b200._nnx_impl import wkv_state_scan

pytestmark = pytest.mark.gpu

TOL = 2e-5


def make_inputs(bsz, steps, n_head, seed, head_dim=64):
    """Inputs with the ranges TimeMix produces: decay = exp(-exp(d)) in (0,1), iclr = sigmoid(.), removal_k
    unit-normalised per head, replacement_k = lerp(k, k*iclr, mix)."""
    rng = np.random.default_rng(seed)
    chans = n_head * head_dim
    shape = (bsz, steps, chans)
    d = rng.standard_normal(shape).astype(np.float32) * 0.5 - 1.0
    decay = np.exp(-np.exp(d)).astype(np.float32)
    iclr = (1.0 / (1.0 + np.exp(-rng.standard_normal(shape)))).astype(np.float32)
    k = rng.standard_normal(shape).astype(np.float32)
    rk = k.reshape(bsz, steps, n_head, head_dim)
    removal_k = (rk / np.maximum(np.linalg.norm(rk, axis=-1, keepdims=True), 1e-12)).reshape(shape).astype(np.float32)
    mix = rng.random(chans).astype(np.float32)
    replacement_k = (k + (k * iclr - k) * mix).astype(np.float32)
    v = rng.standard_normal(shape).astype(np.float32)
    r = rng.standard_normal(shape).astype(np.float32)
    state = (rng.standard_normal((bsz, n_head, head_dim, head_dim)) * 0.1).astype(np.float32)
    return state, decay, iclr, removal_k, replacement_k, v, r


@pytest.mark.parametrize("bsz,steps,n_head,with_state", [(2, 64, 3, True), (1, 7, 1, False), (3, 257, 2, True), (1, 4096, 2, True)])
def test_wkv7_scan_matches_the_oracle(built_lib, bsz, steps, n_head, with_state):
    state, *ins = make_inputs(bsz, steps, n_head, seed=steps)
    s0 = state if with_state else np.zeros_like(state)
    want_state, want_out = wkv7_oracle.wkv_state_scan(s0, *ins, n_head, dtype=np.float64)
    got_state, got_out = wkv_state_scan(torch.from_numpy(s0).cuda() if with_state else None, *[torch.from_numpy(a).cuda() for a in ins], n_head)
    assert got_out.shape == (bsz, steps, n_head * 64) and got_state.shape == (bsz, n_head, 64, 64)
    err_out = np.abs(got_out.cpu().numpy() - want_out).max() / np.abs(want_out).max()
    err_state = np.abs(got_state.cpu().numpy() - want_state).max() / np.abs(want_state).max()
    print(f"B={bsz} T={steps} N={n_head}: out error {err_out:.2e}, state error {err_state:.2e} of the maximum")
    assert err_out <= TOL and err_state <= TOL
    if steps <= 300:        # the oracle in the reference's own precision meets the same bound
        f32_state, f32_out = wkv7_oracle.wkv_state_scan(s0, *ins, n_head, dtype=np.float32)
        assert np.abs(f32_out - want_out).max() / np.abs(want_out).max() <= TOL


def test_wkv7_scan_continues_from_its_own_state(built_lib):
    """Two halves chained through the returned state give the bits of one pass over the whole sequence."""
    state, *ins = make_inputs(2, 128, 2, seed=9)
    t = [torch.from_numpy(a).cuda() for a in ins]
    s_full, y_full = wkv_state_scan(torch.from_numpy(state).cuda(), *t, 2)
    s_half, y_a = wkv_state_scan(torch.from_numpy(state).cuda(), *[a[:, :64].contiguous() for a in t], 2)
    s_end, y_b = wkv_state_scan(s_half, *[a[:, 64:].contiguous() for a in t], 2)
    assert torch.equal(torch.cat([y_a, y_b], dim=1), y_full) and torch.equal(s_end, s_full)


def test_wkv7_scan_rejects_bad_arguments(built_lib):
    z = torch.zeros(1, 4, 96, device="cuda")
    with pytest.raises(Exception):
        wkv_state_scan(None, z, z, z, z, z, z, 2)          # head size 48: the kernel is built for 64
    with pytest.raises(ValueError):
        wkv_state_scan(None, z, z, z, z, z, z[:, :2], 1)
    with pytest.raises(RuntimeError):
        wkv_state_scan(None, *[torch.zeros(1, 4, 64)] * 6, 1)


def _torch_reference(state, ins, n_head):
    """The reference recurrence on torch CPU tensors in float64, differentiated by torch.autograd: an independent
    check of the backward kernel's hand-derived cotangents."""
    decay, iclr, removal_k, replacement_k, v, r = ins
    bsz, steps, chans = decay.shape
    h = chans // n_head
    S = state
    outs = []
    col = lambda a, t: a[:, t].reshape(bsz, n_head, h, 1)
    for t in range(steps):
        w, a, kap, kt, vt, rt = (col(x, t) for x in (decay, iclr, removal_k, replacement_k, v, r))
        S = S * w.mT - S @ kap @ (a * kap).mT
        S = S + vt @ kt.mT
        outs.append((S @ rt).reshape(bsz, chans))
    return S, torch.stack(outs, dim=1)


@pytest.mark.parametrize("bsz,steps,n_head,with_state", [(2, 40, 2, True), (1, 16, 1, False), (2, 97, 3, True), (1, 3, 1, True), (2, 6, 2, False), (1, 13, 2, True), (1, 8, 1, True)])
def test_wkv7_scan_gradients_match_autograd_of_the_reference_recurrence(built_lib, bsz, steps, n_head, with_state):
    """pb_wkv7_backward (checkpoints every 8 timesteps, recomputation in between; the step counts cover full chunks and
    tails of 1 to 7 timesteps) against torch.autograd in float64
    on the CPU; tolerance 1e-4 of each gradient's largest magnitude (fp32 sums of up to 64 terms per timestep,
    chained over the sequence)."""
    state, *ins = make_inputs(bsz, steps, n_head, seed=100 + steps)
    rng = np.random.default_rng(steps)
    g_out = rng.standard_normal((bsz, steps, n_head * 64)).astype(np.float32)
    g_state = rng.standard_normal(state.shape).astype(np.float32) * 0.1
    # reference
    ref_ins = [torch.from_numpy(a).double().requires_grad_(True) for a in ins]
    ref_state = torch.from_numpy(state).double().requires_grad_(True) if with_state else torch.zeros(state.shape, dtype=torch.float64)
    rs, ro = _torch_reference(ref_state, ref_ins, n_head)
    ((ro * torch.from_numpy(g_out).double()).sum() + (rs * torch.from_numpy(g_state).double()).sum()).backward()
    # kernels
    dev_ins = [torch.from_numpy(a).cuda().requires_grad_(True) for a in ins]
    dev_state = torch.from_numpy(state).cuda().requires_grad_(True) if with_state else None
    ds, do = wkv_state_scan(dev_state, *dev_ins, n_head)
    ((do * torch.from_numpy(g_out).cuda()).sum() + (ds * torch.from_numpy(g_state).cuda()).sum()).backward()
    names = ["decay", "iclr", "removal_k", "replacement_k", "v", "r"]
    for name, got, want in zip(names, dev_ins, ref_ins):
        err = (got.grad.cpu().double() - want.grad).abs().max().item() / want.grad.abs().max().item()
        print(f"d{name}: {err:.2e}")
        assert err <= 1e-4, f"gradient of {name} differs by {err:.2e} of its maximum"
    if with_state:
        err = (dev_state.grad.cpu().double() - ref_state.grad).abs().max().item() / ref_state.grad.abs().max().item()
        assert err <= 1e-4, f"gradient of the initial state differs by {err:.2e}"
    # the forward values of the differentiable path are those of the plain path
    with torch.no_grad():
        s2, o2 = wkv_state_scan(dev_state, *dev_ins, n_head)
    assert torch.equal(o2, do) and torch.equal(s2, ds)
