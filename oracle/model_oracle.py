"""CPU restatement (numpy) of the quantized modified-RWKV-7 forward pass of the reference: the layers of
pratchya/_nnx_impl/_module.py and the model and loss of _model.py / _utils.py, on top of the quantization
oracle (qarr_oracle) and the scan oracle (wkv7_oracle).

TEST INFRASTRUCTURE ONLY: the parity checker of pratchya_b200/_nnx_impl/_model.py.  Nothing in the shipped package
imports it.

PARITY UNPINNED: the reference has no tests or vectors for these layers and cannot be imported here (jax and flax
are not installed).  Each function cites the reference lines it follows.  Parameters come in as a dict of numpy
arrays keyed like the torch module's state_dict (dense values; a quantized parameter of the reference reads as
dequantize(quantize(value)), which `read` applies)."""
from __future__ import annotations

import numpy as np

from . import qarr_oracle as q
from . import wkv7_oracle

F32 = np.float32


def read(p, tgrid):
    """`QArrayImpl(p, tgrid).astype(f32)`: _qarr.py:29, :339-342."""
    p = np.asarray(p, dtype=F32)
    return q.dequantize_nd(*q.quantize_nd(p, tgrid), F32, tgrid)


def linear(x, kernel, tgrid):
    """Linear.__call__, _module.py:46-50."""
    x = np.asarray(x, dtype=F32)
    lead = x.shape[:-1]
    y = q.linear_forward(x.reshape(-1, x.shape[-1]), q.quantize_impl(np.asarray(kernel, dtype=F32), tgrid), tgrid)
    return y.reshape(*lead, kernel.shape[1])


def lerp(i, j, w):                                   # _module.py:12-13
    return (i + (j - i) * w).astype(F32)


def normalized(x, axis, eps=1e-12):                  # _module.py:15-18
    return (x / np.sqrt(np.sum(np.square(x), axis=axis, keepdims=True) + F32(eps))).astype(F32)


def sigmoid(x):
    return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(F32)


def low_rank_ffn(x, p, prefix, blk):                 # _module.py:74-89
    return linear(np.tanh(linear(x, p[prefix + ".down.kernel"], (blk, 1))).astype(F32), p[prefix + ".up.kernel"], (blk, 1))


def rms_norm(x, scale, blk, eps):                    # _module.py:61-72
    x = x.astype(F32)
    inv = 1.0 / np.sqrt(np.mean(np.square(x), axis=-1, keepdims=True) + F32(eps))
    return (x * inv.astype(F32) * read(scale, (1, blk))).astype(F32)


def rotary(x, t, head_dim, theta):                   # _module.py:261-283; x [B, T, N, H]
    inv_freq = (1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=F32) / F32(head_dim)))).astype(F32)
    freqs = np.outer(t.astype(F32), inv_freq).astype(F32)
    emb = np.concatenate([freqs, freqs], axis=-1)[:, None, :]
    d = x.shape[-1]
    rotated = np.concatenate([-x[..., d // 2:], x[..., : d // 2]], axis=-1)
    return (x * np.cos(emb) + rotated * np.sin(emb)).astype(F32)


def group_norm(x, n_groups, eps, scale, bias):
    """flax.nnx.GroupNorm as TimeMix builds it (_module.py:118-123) on [B, T, C]: statistics per batch element and group
    over the T positions and the group's channels, variance as E[x^2] - E[x]^2."""
    b, t, c = x.shape
    g = x.reshape(b, t, n_groups, c // n_groups).astype(F32)
    mean = g.mean(axis=(1, 3), keepdims=True)
    var = np.maximum((g * g).mean(axis=(1, 3), keepdims=True) - mean * mean, 0.0)
    out = ((g - mean) / np.sqrt(var + F32(eps))).reshape(b, t, c)
    return (out * scale + bias).astype(F32)


def time_mix(x, v_prime_0, t_positions, tm_state, wkv_state, p, pre, cfg, first_layer):
    """TimeMix.__call__, _module.py:129-225."""
    b, t, c = x.shape
    h = cfg["head_dim"]
    n = c // h
    blk = cfg["blksize"]
    x_shifted = np.concatenate([tm_state, x[:, :-1, :]], axis=1)
    mu = read(p[pre + ".mu"], (1, blk))
    xr, xd, xk, xv, xi, xg = (lerp(x, x_shifted, mu[j]) for j in range(6))
    grid = (blk, blk)
    r = linear(xr, p[pre + ".w_receptance.kernel"], grid)
    d = low_rank_ffn(xd, p, pre + ".decay_lora", blk)
    k = linear(xk, p[pre + ".w_key.kernel"], grid)
    v_prime = linear(xv, p[pre + ".w_value.kernel"], grid)
    gate = low_rank_ffn(xg, p, pre + ".gate_lora", blk)
    iclr = sigmoid(low_rank_ffn(xi, p, pre + ".iclr_lora", blk))
    k = rotary(k.reshape(b, t, n, h), t_positions, h, cfg["rope_theta"]).reshape(b, t, c)
    r = rotary(r.reshape(b, t, n, h), t_positions, h, cfg["rope_theta"]).reshape(b, t, c)
    if first_layer:
        v = v_prime_0 = v_prime
    else:
        nu = sigmoid(low_rank_ffn(xv, p, pre + ".nu_lora", blk))
        v = lerp(v_prime, v_prime_0, nu)
    decay = np.exp(-np.exp(d.astype(np.float64))).astype(F32)
    removal_k = (k * read(p[pre + ".removal_key_multiplier"], (1, blk))).astype(F32)
    removal_k = normalized(removal_k.reshape(b, t, n, h), axis=-1).reshape(b, t, c)
    replacement_k = lerp(k, (k * iclr).astype(F32), read(p[pre + ".iclr_mix_amt"], (1, blk)))
    wkv_state, out = wkv7_oracle.wkv_state_scan(wkv_state, decay, iclr, removal_k, replacement_k, v, r, n, dtype=F32)
    out = group_norm(out, n, n * 1e-5, p[pre + ".gn_scale"], p[pre + ".gn_bias"])
    bonus = (np.sum(r * k * read(p[pre + ".bonus_multiplier"], (1, blk)), axis=-1, keepdims=True) * v).astype(F32)
    out = ((out + bonus) * gate).astype(F32)
    return linear(out, p[pre + ".w_output.kernel"], grid), v, x[:, -1:, :], wkv_state


def channel_mix(x, cm_state, p, pre, cfg):
    """ChannelMix.__call__, _module.py:236-258."""
    blk = cfg["blksize"]
    x_shifted = np.concatenate([cm_state, x[:, :-1, :]], axis=1)
    xk = lerp(x, x_shifted, read(p[pre + ".mu_x"], (1, blk)))
    k = linear(xk, p[pre + ".w_k.kernel"], (blk, blk))
    k = (np.maximum(k, 0) ** 2).astype(F32)
    return linear(k, p[pre + ".w_v.kernel"], (blk, blk)), x[:, -1:, :]


def block(x, v_0, t_positions, p, pre, cfg, first_layer):
    """RWKVBlock.__call__, _module.py:300-317, from zero states."""
    b, _, c = x.shape
    h = cfg["head_dim"]
    zeros = np.zeros((b, 1, c), dtype=F32)
    x = rms_norm(x, p[pre + ".pre_rmsnorm.scale"], cfg["blksize"], cfg["rmsnorm_epsilon"])
    dx, v_0, _, _ = time_mix(x, v_0, t_positions, zeros, np.zeros((b, c // h, h, h), dtype=F32), p, pre + ".tm", cfg, first_layer)
    x = (x + dx).astype(F32)
    x = rms_norm(x, p[pre + ".post_rmsnorm.scale"], cfg["blksize"], cfg["rmsnorm_epsilon"])
    dx, _ = channel_mix(x, zeros, p, pre + ".cm", cfg)
    return (x + dx).astype(F32), v_0


def causal_lm(input_ids, labels, p, cfg):
    """PratchyaCausalLM.__call__ with PratchyaModel inside, _model.py:43-96, and compute_loss, _utils.py:7-13."""
    b, t = input_ids.shape
    blk = cfg["blksize"]
    x = (read(p["embedding"][input_ids], (1, blk)) * F32(np.sqrt(cfg["hidden_size"]))).astype(F32)      # EmbeddingScaled, _module.py:32-37
    x = rms_norm(x, p["pre_rmsnorm.scale"], blk, cfg["rmsnorm_epsilon"])
    t_positions = np.arange(t, dtype=np.int32)
    v = None
    for i in range(cfg["n_layers"]):
        x, v = block(x, v, t_positions, p, f"blocks.{i}", cfg, first_layer=i == 0)
    x = rms_norm(x, p["final_rmsnorm.scale"], blk, cfg["rmsnorm_epsilon"])
    logits = linear(x, p["lm_head.kernel"], (blk, 1))
    loss = None
    if labels is not None:
        lg = logits[:, :-1, :].astype(np.float64)
        lb = labels[:, 1:]
        logp = lg - lg.max(axis=-1, keepdims=True)
        logp = logp - np.log(np.exp(logp).sum(axis=-1, keepdims=True))
        n_cls = lg.shape[-1]
        one_hot = np.eye(n_cls)[lb]
        smoothed = (1.0 - 0.1) * one_hot + 0.1 / n_cls                                                 # optax.smooth_labels
        loss = float(np.mean(-(smoothed * logp).sum(axis=-1)))
    return logits, loss
