"""CPU checks of oracle/model_oracle.py (the numpy restatement of the quantized modified RWKV-7 forward pass) through
properties the reference's text implies: causality of ChannelMix's token shift, the loss formula, GroupNorm's
statistics, and what a read of a quantized parameter returns."""
import numpy as np

from oracle import model_oracle as mo
from oracle import qarr_oracle as q

CFG = dict(vocab_size=256, hidden_size=1024, intermediate_size=1024, lora_rank=128, head_dim=64, n_layers=2, blksize=128,
           rmsnorm_epsilon=1e-6, rope_theta=1e4)


def make_params(seed=0):
    rng = np.random.default_rng(seed)
    c, f, r, v = CFG["hidden_size"], CFG["intermediate_size"], CFG["lora_rank"], CFG["vocab_size"]
    n = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)
    p = {"embedding": n(v, c, scale=c ** -0.5), "pre_rmsnorm.scale": np.ones((1, c), np.float32),
         "final_rmsnorm.scale": np.ones((1, c), np.float32), "lm_head.kernel": n(c, v, scale=c ** -0.5)}
    for i in range(CFG["n_layers"]):
        b = f"blocks.{i}"
        p[f"{b}.pre_rmsnorm.scale"] = np.ones((1, c), np.float32)
        p[f"{b}.post_rmsnorm.scale"] = np.ones((1, c), np.float32)
        p[f"{b}.tm.mu"] = n(6, c, scale=0.4)
        for w in ("w_key", "w_value", "w_output", "w_receptance"):
            p[f"{b}.tm.{w}.kernel"] = n(c, c, scale=c ** -0.5)
        for lora in ("gate_lora", "decay_lora", "iclr_lora") + (("nu_lora",) if i > 0 else ()):
            p[f"{b}.tm.{lora}.down.kernel"] = n(c, r, scale=c ** -0.5)
            p[f"{b}.tm.{lora}.up.kernel"] = n(r, c, scale=r ** -0.5)
        for name in ("iclr_mix_amt", "removal_key_multiplier", "bonus_multiplier"):
            p[f"{b}.tm.{name}"] = n(1, c)
        p[f"{b}.tm.gn_scale"] = np.ones(c, np.float32)
        p[f"{b}.tm.gn_bias"] = np.zeros(c, np.float32)
        p[f"{b}.cm.w_k.kernel"] = n(c, f, scale=c ** -0.5)
        p[f"{b}.cm.w_v.kernel"] = n(f, c, scale=f ** -0.5)
        p[f"{b}.cm.mu_x"] = n(1, c, scale=0.4)
    return p


def test_read_is_quantize_then_dequantize():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((1, 256)).astype(np.float32)
    assert np.array_equal(mo.read(w, (1, 128)), q.dequantize_impl(*q.quantize_impl(w, (1, 128)), np.float32, (1, 128)))


def test_channel_mix_is_causal_and_uses_the_carried_token():
    """With 1024 channels every (1,128) super-group of eight blocks lies inside one token's row, so ChannelMix is causal.
    (With fewer than eight blocks per row the reference's super-groups span neighbouring tokens and couple them through
    the shared fp32 amax: that is its rule, and the reason this test uses 1024 channels.)"""
    p = make_params()
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1, 6, CFG["hidden_size"])).astype(np.float32)
    state = rng.standard_normal((1, 1, CFG["hidden_size"])).astype(np.float32)
    out, carried = mo.channel_mix(x, state, p, "blocks.0.cm", CFG)
    assert np.array_equal(carried, x[:, -1:, :])
    x2 = x.copy()
    x2[:, 4:, :] += 1.0                                         # a change at position 4 leaves positions 0..3 alone
    out2, _ = mo.channel_mix(x2, state, p, "blocks.0.cm", CFG)
    assert np.array_equal(out[:, :4], out2[:, :4]) and not np.array_equal(out[:, 4:], out2[:, 4:])
    out3, _ = mo.channel_mix(x, state * 0, p, "blocks.0.cm", CFG)   # the carried token reaches position 0 only
    assert not np.array_equal(out[:, 0], out3[:, 0]) and np.array_equal(out[:, 1:], out3[:, 1:])


def test_group_norm_statistics_span_time_and_the_groups_channels():
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((2, 5, 128)) * 3 + 1).astype(np.float32)
    out = mo.group_norm(x, 2, 2e-5, np.ones(128, np.float32), np.zeros(128, np.float32))     # two groups of 64 channels
    g = out.reshape(2, 5, 2, 64)
    assert np.allclose(g.mean(axis=(1, 3)), 0.0, atol=1e-5) and np.allclose(g.var(axis=(1, 3)), 1.0, atol=1e-3)


def test_model_runs_and_the_loss_is_the_smoothed_cross_entropy():
    p = make_params()
    rng = np.random.default_rng(4)
    ids = rng.integers(0, CFG["vocab_size"], (1, 8))
    logits, loss = mo.causal_lm(ids, ids, p, CFG)
    assert logits.shape == (1, 8, CFG["vocab_size"]) and np.isfinite(logits).all()
    # (No causality check here: GroupNorm's statistics span the whole sequence -- flax GroupNorm on [B, T, C] -- and the
    # rank-128 LoRA activations are quantized in super-groups of several tokens, so the model as the reference writes it
    # lets a later token move earlier logits, and on a sequence this short it moves them as much as the later ones.)
    # loss by hand
    lg = logits[:, :-1].astype(np.float64)
    logp = lg - np.log(np.exp(lg - lg.max(-1, keepdims=True)).sum(-1, keepdims=True)) - lg.max(-1, keepdims=True)
    tgt = ids[:, 1:]
    nll = -np.take_along_axis(logp, tgt[..., None], -1)[..., 0]
    want = np.mean(0.9 * nll + 0.1 * (-logp.mean(-1)))
    assert abs(loss - want) <= 1e-9
