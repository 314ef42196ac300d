"""The fused element-wise kernels of the RWKV-7 block (csrc/rwkv_glue.cu through pratchya_b200/_nnx_impl/_glue.py)
against the same formulas evaluated operation by operation in torch f32 (the text of the reference's TimeMix and
ChannelMix, pratchya/_nnx_impl/_module.py:129-258), values and gradients.

Forward values: bit-equal where the kernel performs the same f32 operations in the same order (lerps, rotary
embedding, sigmoid, exp); 1e-6 of the largest magnitude where a 64-term sum is formed in another order (normalized).
Gradients: 2e-5 of each gradient's largest magnitude against torch.autograd (sums over tokens in another order)."""
import pytest
import torch

from pratchya_b200._nnx_impl._glue import token_shift_lerp, token_shift_lerp_quantized, wkv_prepare
from pratchya_b200._nnx_impl._model import PratchyaCausalLM, PratchyaConfig, lerp, normalized, RotaryEmbedding

pytestmark = pytest.mark.gpu


def close(got, want, what, tol):
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    assert err <= tol * max(scale, 1e-30), f"{what}: error {err:.3e} against a largest magnitude of {scale:.3e}"


@pytest.mark.parametrize("bsz,steps,chans,n_mix,with_state", [(2, 37, 1024, 6, True), (3, 300, 2048, 1, True), (1, 513, 1024, 6, False),
                                                              (2, 256, 2048, 6, True), (5, 1, 1024, 1, True)])
def test_token_shift_lerp_matches_torch(built_lib, bsz, steps, chans, n_mix, with_state):
    gen = torch.Generator(device="cuda").manual_seed(steps + n_mix)
    x = torch.randn(bsz, steps, chans, device="cuda", generator=gen).requires_grad_(True)
    state = torch.randn(bsz, 1, chans, device="cuda", generator=gen).requires_grad_(True) if with_state else None
    mu = torch.randn(n_mix, chans, device="cuda", generator=gen).requires_grad_(True)
    g = torch.randn(n_mix, bsz, steps, chans, device="cuda", generator=gen)
    got = torch.stack(token_shift_lerp(x, state, mu))
    first = state if with_state else torch.zeros(bsz, 1, chans, device="cuda")
    shifted = torch.cat([first, x[:, :-1, :]], dim=1)
    want = torch.stack([lerp(x, shifted, mu[k]) for k in range(n_mix)])
    assert torch.equal(got, want)
    leaves = [x, mu] + ([state] if with_state else [])
    got_grads = torch.autograd.grad(got, leaves, g)
    want_grads = torch.autograd.grad(want, leaves, g)
    for name, a, b in zip(["dx", "dmu", "dstate"], got_grads, want_grads):
        close(a, b, name, 2e-5)


@pytest.mark.parametrize("bsz,steps,chans,n_mix,with_state,transposed", [
    (2, 37, 1024, 6, True, ()), (1, 300, 2048, 1, False, ()),                    # row forms only (any number of steps)
    (2, 1024, 1024, 6, True, (0, 2, 3)), (3, 2048, 2048, 1, True, (0,)),         # with token-major forms; fewer tiles than SMs, then more
    (2, 1024, 2048, 6, False, (5,)), (5, 1024, 1024, 6, True, (0, 1, 2, 3, 4, 5))])
def test_token_shift_lerp_quantized_gives_the_bytes_of_lerp_then_quantize(built_lib, bsz, steps, chans, n_mix, with_state, transposed):
    """The lerp fused into the activation quantizers: every triple bit for bit that of the quantizer run on the mix
    the unfused kernel writes (which the test above checks against torch), in the row form and in the token-major
    form; sequences start at tile boundaries, inside the array too (bsz > 1), with and without a carried state.
    Gradients flow through the storage-less handles to x, state and mu as they do through the unfused mixes."""
    from pratchya_b200 import _lib
    from pratchya_b200._qualia import quantize_impl, quantize_transposed_impl
    from pratchya_b200._nnx_impl import linear_fp8
    gen = torch.Generator(device="cuda").manual_seed(steps + 7 * n_mix)
    x = torch.randn(bsz, steps, chans, device="cuda", generator=gen)
    x.view(-1)[::4099] *= 50.0
    x[0, : min(steps, 1024), 3] = 0.0                              # an all-zero token-major super-group when mu or the state is zero there
    state = torch.randn(bsz, 1, chans, device="cuda", generator=gen) if with_state else None
    mu = torch.rand(n_mix, chans, device="cuda", generator=gen)
    mu[:, 3] = 0.0
    mixes = token_shift_lerp_quantized(x, state, mu, transposed)
    torch.cuda.synchronize()
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    plain = token_shift_lerp(x, state, mu)
    as_bytes = lambda t: t.contiguous().view(torch.uint8)
    for k in range(n_mix):
        v = plain[k].reshape(-1, chans)
        for got, want in zip(mixes[k].row, quantize_impl(v, (1, 128))):
            assert got.shape == want.shape and torch.equal(as_bytes(got), as_bytes(want)), f"row form of mix {k}"
        if k in transposed:
            for got, want in zip(mixes[k].tokens, quantize_transposed_impl(v, 128)):
                assert got.shape == want.shape and torch.equal(as_bytes(got), as_bytes(want)), f"token-major form of mix {k}"
        else:
            assert mixes[k].tokens is None
    # through a Linear: same output, same gradients as the unfused chain
    if transposed:
        w = (torch.randn(chans, 256, device="cuda", generator=gen) * 0.03).requires_grad_(True)
        g = torch.randn(bsz, steps, 256, device="cuda", generator=gen)
        k = transposed[0]
        results = []
        for fused in (True, False):
            xx, mm = x.clone().requires_grad_(True), mu.clone().requires_grad_(True)
            ss = state.clone().requires_grad_(True) if with_state else None
            mix = (token_shift_lerp_quantized(xx, ss, mm, transposed) if fused else token_shift_lerp(xx, ss, mm))[k]
            y = linear_fp8(mix, w, (128, 128))
            grads = torch.autograd.grad(y, [xx, mm, w] + ([ss] if with_state else []), g)
            results.append((y.detach(), grads))
        assert torch.equal(results[0][0], results[1][0])
        for a, b in zip(results[0][1], results[1][1]):
            assert torch.equal(a, b)


@pytest.mark.parametrize("bsz,steps,n_head,first_layer", [(2, 33, 4, True), (2, 200, 3, False), (1, 129, 32, False)])
def test_wkv_prepare_matches_torch(built_lib, bsz, steps, n_head, first_layer):
    gen = torch.Generator(device="cuda").manual_seed(steps)
    c = n_head * 64
    mk = lambda scale=1.0: (torch.randn(bsz, steps, c, device="cuda", generator=gen) * scale).requires_grad_(True)
    r_raw, k_raw, d, iclr_raw, v_prime = mk(), mk(), mk(0.5), mk(), mk()
    v0, nu_raw = (None, None) if first_layer else (mk(), mk())
    rk_mult = torch.randn(1, c, device="cuda", generator=gen).requires_grad_(True)
    mix_amt = torch.randn(1, c, device="cuda", generator=gen).requires_grad_(True)
    cfg = PratchyaConfig()
    rotary = RotaryEmbedding(cfg, "cuda")
    t = torch.arange(steps, device="cuda", dtype=torch.int32)
    cos_tab, sin_tab = rotary.tables(t)
    got = wkv_prepare(r_raw, k_raw, d, iclr_raw, v_prime, v0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt, n_head)

    k = rotary(k_raw.reshape(bsz, steps, n_head, 64), t).reshape(bsz, steps, c)
    r = rotary(r_raw.reshape(bsz, steps, n_head, 64), t).reshape(bsz, steps, c)
    iclr = torch.sigmoid(iclr_raw)
    v = v_prime if first_layer else lerp(v_prime, v0, torch.sigmoid(nu_raw))
    decay = torch.exp(-torch.exp(d))
    removal_k = normalized((k * rk_mult).reshape(bsz, steps, n_head, 64), dim=-1).reshape(bsz, steps, c)
    replacement_k = lerp(k, k * iclr, mix_amt)
    want = (decay, iclr, removal_k, replacement_k, v, r, k)
    names = ["decay", "iclr", "removal_k", "replacement_k", "v", "r", "k"]
    for name, a, b in zip(names, got, want):
        if name == "removal_k":
            close(a, b, name, 1e-6)
        elif name in ("decay", "iclr", "replacement_k", "v"):      # through exp / sigmoid: the same library functions, allow an ulp
            close(a, b, name, 3e-7)
        else:
            assert torch.equal(a, b), name
    leaves = [r_raw, k_raw, d, iclr_raw, v_prime, rk_mult, mix_amt] + ([] if first_layer else [v0, nu_raw])
    gs = [torch.randn(bsz, steps, c, device="cuda", generator=gen) for _ in range(7)]
    got_grads = torch.autograd.grad(got, leaves, gs)
    want_grads = torch.autograd.grad(want, leaves, gs)
    leaf_names = ["d_r_raw", "d_k_raw", "d_d", "d_iclr_raw", "d_v_prime", "d_rk_mult", "d_mix_amt", "d_v0", "d_nu_raw"]
    for name, a, b in zip(leaf_names, got_grads, want_grads):
        close(a, b, name, 2e-5)


def test_model_with_fused_glue_matches_the_op_by_op_model(built_lib):
    kw = dict(vocab_size=1024, hidden_size=1024, intermediate_size=2048, n_layers=2)
    fused = PratchyaCausalLM(PratchyaConfig(fused_glue=True, **kw), seed=3, remat=False)
    plain = PratchyaCausalLM(PratchyaConfig(fused_glue=False, **kw), seed=3, remat=False)
    plain.load_state_dict(fused.state_dict())
    gen = torch.Generator(device="cuda").manual_seed(4)
    ids = torch.randint(0, 1024, (2, 48), device="cuda", generator=gen)
    logits_f, loss_f = fused(ids, ids)
    logits_p, loss_p = plain(ids, ids)
    # the products are re-quantized to fp8 after every linear: an ulp of difference in a 64-term sum moves a rounding
    # now and then, so the comparison is statistical, as between the device and the oracle
    diff = (logits_f - logits_p).abs()
    scale = logits_p.abs().max()
    print(f"logits: mean difference {diff.mean() / scale:.2e}, largest {diff.max() / scale:.2e}; loss {loss_f.item():.5f} vs {loss_p.item():.5f}")
    assert diff.mean() <= 6e-3 * scale and abs(loss_f.item() - loss_p.item()) <= 5e-3
    loss_f.backward()
    loss_p.backward()
    for (name, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        assert a.grad is not None and torch.isfinite(a.grad).all(), name
        cos = torch.nn.functional.cosine_similarity(a.grad.flatten(), b.grad.flatten(), dim=0).item()
        assert cos > 0.98, f"gradient of {name}: cosine {cos:.4f} between the fused and the op-by-op model"


@pytest.mark.parametrize("shape", [(3, 50, 1024), (700, 2048), (2, 4096, 128)])
def test_rms_norm_matches_torch(built_lib, shape):
    from pratchya_b200._nnx_impl._glue import rms_norm
    gen = torch.Generator(device="cuda").manual_seed(shape[-1] + shape[0])
    x = (torch.randn(*shape, device="cuda", generator=gen) * 3).requires_grad_(True)
    scale = (1 + 0.1 * torch.randn(1, shape[-1], device="cuda", generator=gen)).requires_grad_(True)
    g = torch.randn(*shape, device="cuda", generator=gen)
    got = rms_norm(x, scale, 1e-6)
    want = x * torch.rsqrt(torch.mean(torch.square(x), dim=-1, keepdim=True) + 1e-6) * scale
    close(got, want, "rms_norm", 5e-7)
    for name, a, b in zip(["dx", "dscale"], torch.autograd.grad(got, [x, scale], g), torch.autograd.grad(want, [x, scale], g)):
        close(a, b, name, 2e-5)


@pytest.mark.parametrize("shape", [(1024, 1024), (2, 1024, 2048), (8, 512, 8192)])
def test_relu2_quantized_gives_the_bytes_of_relu2_then_quantize(built_lib, shape):
    """relu^2 as the prologue of the row and the token-major quantizer: byte for byte the triples of the quantizers run on
    the array the relu2 kernel writes, and the same gradient through a Linear."""
    from pratchya_b200 import _lib
    from pratchya_b200._qualia import quantize_impl, quantize_transposed_impl
    from pratchya_b200._nnx_impl import linear_fp8
    from pratchya_b200._nnx_impl._glue import relu2, relu2_quantized
    gen = torch.Generator(device="cuda").manual_seed(sum(shape))
    k = torch.randn(shape, device="cuda", generator=gen) * 2.0
    k.view(-1)[::4099] *= 40.0
    mix = relu2_quantized(k)
    torch.cuda.synchronize()
    _lib.check(built_lib.pb_gemm_check(torch.cuda.current_stream().cuda_stream))
    k2 = relu2(k).reshape(-1, shape[-1])
    as_bytes = lambda t: t.contiguous().view(torch.uint8)
    for got, want in zip(mix.row, quantize_impl(k2, (1, 128))):
        assert got.shape == want.shape and torch.equal(as_bytes(got), as_bytes(want))
    for got, want in zip(mix.tokens, quantize_transposed_impl(k2, 128)):
        assert got.shape == want.shape and torch.equal(as_bytes(got), as_bytes(want))
    w = (torch.randn(shape[-1], 256, device="cuda", generator=gen) * 0.03).requires_grad_(True)
    g = torch.randn(*shape[:-1], 256, device="cuda", generator=gen)
    results = []
    for fused in (True, False):
        kk = k.clone().requires_grad_(True)
        y = linear_fp8(relu2_quantized(kk) if fused else relu2(kk), w, (128, 128))
        results.append((y.detach(), torch.autograd.grad(y, [kk, w], g)))
    assert torch.equal(results[0][0], results[1][0])
    for a, b in zip(results[0][1], results[1][1]):
        assert torch.equal(a, b)


def test_relu2_matches_torch(built_lib):
    from pratchya_b200._nnx_impl._glue import relu2
    gen = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(3, 77, 2048, device="cuda", generator=gen).requires_grad_(True)
    g = torch.randn(3, 77, 2048, device="cuda", generator=gen)
    got, want = relu2(x), torch.relu(x) ** 2
    assert torch.equal(got, want)
    assert torch.equal(torch.autograd.grad(got, x, g)[0], torch.autograd.grad(want, x, g)[0])


@pytest.mark.parametrize("bsz,steps,n_head", [(2, 33, 4), (2, 300, 3), (1, 520, 32)])
def test_wkv_finish_matches_torch(built_lib, bsz, steps, n_head):
    from pratchya_b200._nnx_impl._glue import wkv_finish
    from pratchya_b200._nnx_impl._model import group_norm
    gen = torch.Generator(device="cuda").manual_seed(steps)
    c = n_head * 64
    mk = lambda: torch.randn(bsz, steps, c, device="cuda", generator=gen).requires_grad_(True)
    y, r, k, v, gate = mk(), mk(), mk(), mk(), mk()
    with torch.no_grad():
        y.mul_(2.0).add_(0.3)
    gs = (1 + 0.1 * torch.randn(c, device="cuda", generator=gen)).requires_grad_(True)
    gb = (0.1 * torch.randn(c, device="cuda", generator=gen)).requires_grad_(True)
    bm = (0.05 * torch.randn(1, c, device="cuda", generator=gen)).requires_grad_(True)
    eps = n_head * 1e-5
    got = wkv_finish(y, r, k, v, gate, gs, gb, bm, eps, n_head)
    want = (group_norm(y, n_head, eps, gs, gb) + torch.sum(r * k * bm, dim=-1, keepdim=True) * v) * gate
    close(got, want, "wkv_finish", 2e-6)
    g = torch.randn(bsz, steps, c, device="cuda", generator=gen)
    leaves = [y, r, k, v, gate, gs, gb, bm]
    for name, a, b in zip(["d_y", "d_r", "d_k", "d_v", "d_gate", "d_gn_scale", "d_gn_bias", "d_bonus_mult"],
                          torch.autograd.grad(got, leaves, g), torch.autograd.grad(want, leaves, g)):
        close(a, b, name, 3e-5)


@pytest.mark.parametrize("bsz,steps,vocab", [(2, 9, 1024), (3, 33, 65536), (1, 2, 4)])
def test_fused_cross_entropy_matches_torch(built_lib, bsz, steps, vocab):
    from pratchya_b200._nnx_impl._glue import smoothed_cross_entropy as fused
    from pratchya_b200._nnx_impl._model import smoothed_cross_entropy as plain
    gen = torch.Generator(device="cuda").manual_seed(vocab + steps)
    logits = (torch.randn(bsz, steps, vocab, device="cuda", generator=gen) * 3).requires_grad_(True)
    labels = torch.randint(0, vocab, (bsz, steps), device="cuda", generator=gen)
    got, want = fused(logits, labels), plain(logits, labels)
    assert abs(got.item() - want.item()) <= 2e-6 * abs(want.item()), (got.item(), want.item())
    g_got, = torch.autograd.grad(got * 1.7, logits)
    g_want, = torch.autograd.grad(want * 1.7, logits)
    close(g_got, g_want, "dlogits", 2e-5)
    assert torch.count_nonzero(g_got[:, -1, :]).item() == 0      # the last position predicts nothing
    # the cotangent written over the logits: same bits, in the logits' own memory
    scratch = logits.detach().clone().requires_grad_(True)
    work = scratch * 1.0                                           # a non-leaf array that nothing else reads
    g_inplace, = torch.autograd.grad(fused(work, labels, reuse_logits=True) * 1.7, scratch)
    assert torch.equal(g_inplace, g_got)
