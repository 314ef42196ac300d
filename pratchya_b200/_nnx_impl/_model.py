"""The modified RWKV-7 model of pratchya/_nnx_impl/_module.py and _model.py (quantized variant) with every
linear layer on the FP8 path of this package and the WKV-7 state scan on its CUDA kernels.

This is the caller of the hot path, kept as close to the reference's text as torch allows.  The pieces that carry
the arithmetic are `linear_fp8` (quantize, block-scaled tensor-core matmuls forward and backward), `FakeQuant` (the
quantize -> dequantize a QArrayImpl parameter goes through when it is read, with the reference's cotangent rule) and
`wkv_state_scan`.  The f32 element-wise work between them (token shift, lerps, rotary embedding, gates,
normalisations, the loss) runs on the fused kernels of `_glue.py` by default; `PratchyaConfig.fused_glue=False` runs
the same formulas as plain torch operations differentiated by torch.autograd, which is what the tests compare with.

Parameters are dense master tensors that are quantized on their grid every time they are used (the
benchmark configuration trains bf16/f32 masters); the reference stores the fp8 triple itself as the
parameter, which gives the same forward values."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .._qualia import _ops
from ._glue import QuantizedMix, can_quantize_mixes, can_quantize_relu2, relu2, relu2_quantized, rms_norm, token_shift_lerp, token_shift_lerp_quantized, wkv_finish, wkv_prepare
from ._glue import smoothed_cross_entropy as fused_cross_entropy
from ._module import linear_fp8
from ._wkv7 import wkv_state_scan


@dataclass
class PratchyaConfig:
    """pratchya/_config.py:8-26 (the fields the quantized model reads)."""
    vocab_size: int = 65536
    hidden_size: int = 2048
    intermediate_size: int = 8192
    lora_rank: int = 128
    head_dim: int = 64
    rmsnorm_epsilon: float = 1e-6
    n_layers: int = 24
    blksize: int = 128
    rope_theta: float = 1e4
    fused_glue: bool = True      # the element-wise work on the kernels of _glue.py instead of op-by-op torch (same values)


def lerp(i, j, w):                                   # _module.py:12-13
    return i + (j - i) * w


def normalized(x, dim: int, eps: float = 1e-12):     # _module.py:15-18
    return x / torch.sqrt(torch.sum(torch.square(x), dim=dim, keepdim=True) + eps)


class FakeQuant(torch.autograd.Function):
    """`QArrayImpl(x, tgrid).astype(dtype)`: what a read of a quantized parameter returns (_qarr.py:29, :339-342).
    Backward: the cotangent of dequantize_impl, g * x_sc / 128 (:575-601), which quantize_impl's rule hands on to x
    unchanged (:519-520)."""

    @staticmethod
    def forward(ctx, x, tgrid, dtype):
        q, sc8, sc32 = _ops.quantize_impl(x, tgrid)
        ctx.save_for_backward(sc8, sc32)
        ctx.tgrid, ctx.x_dtype = tgrid, x.dtype
        return _ops.dequantize_impl(q, sc8, sc32, dtype, tgrid)

    @staticmethod
    def backward(ctx, g):
        sc8, sc32 = ctx.saved_tensors
        return _ops.dequantize_impl_bwd(sc8, sc32, g.contiguous(), ctx.tgrid).to(ctx.x_dtype), None, None


def read_param(p, tgrid, dtype=torch.float32):
    return FakeQuant.apply(p, tgrid, dtype)


def _lecun(fan_in, shape, gen, device):
    return torch.randn(shape, generator=gen, device=device) * math.sqrt(1.0 / fan_in)


class Linear(torch.nn.Module):
    """_module.py:39-50 with a dense master kernel: y = dq(q(dq(Q(x,(1,a))) @ dq(Q(W,tgrid)), (1,b))).astype(x.dtype).
    On a (blk,1) grid the product's re-quantization is on (1,1), where every element is its own block and
    dq(q(y)) == y (apart from |y| < 1e-7): it is left out."""

    def __init__(self, fan_in, fan_out, tgrid, gen, device):
        super().__init__()
        self.tgrid = (int(tgrid[0]), int(tgrid[1]))
        self.kernel = torch.nn.Parameter(_lecun(fan_in, (fan_in, fan_out), gen, device))
        self._prepared = (None, None)        # (kernel version, {"wq": fp8 triple, "w_t": its byte transpose})

    def forward(self, x, raw=False):
        """`raw`: return the f32 product itself, without its re-quantization (for a caller that fuses that step
        into what follows)."""
        # the kernel's fp8 form is the same in every pass of a step: keep it until the kernel is written to
        version = (self.kernel._version, self.kernel.data_ptr())
        if self._prepared[0] != version:
            self._prepared = (version, {})
        return linear_fp8(x, self.kernel, self.tgrid, fake_quant_output=self.tgrid[1] != 1 and not raw, prepared=self._prepared[1])


class LowRankFFN(torch.nn.Module):                   # _module.py:74-89
    def __init__(self, hidden, rank, blk, gen, device):
        super().__init__()
        self.down = Linear(hidden, rank, (blk, 1), gen, device)
        self.up = Linear(rank, hidden, (blk, 1), gen, device)

    def forward(self, x):
        return self.up(torch.tanh(self.down(x)))


class RMSNorm(torch.nn.Module):                      # _module.py:61-72
    def __init__(self, hidden, blk, eps, device, fused=True):
        super().__init__()
        self.eps, self.blk, self.fused = eps, blk, fused
        self.scale = torch.nn.Parameter(torch.ones(1, hidden, device=device))

    def forward(self, x):
        if self.fused:
            return rms_norm(x, read_param(self.scale, (1, self.blk)), self.eps).to(x.dtype)
        x32 = x.to(torch.float32)
        inv_rms = torch.rsqrt(torch.mean(torch.square(x32), dim=-1, keepdim=True) + self.eps)
        return (x32 * inv_rms * read_param(self.scale, (1, self.blk))).to(x.dtype)


class RotaryEmbedding(torch.nn.Module):              # _module.py:261-283
    def __init__(self, cfg, device):
        super().__init__()
        h = cfg.head_dim
        self.register_buffer("inv_freq", 1.0 / (cfg.rope_theta ** (torch.arange(0, h, 2, dtype=torch.float32, device=device) / h)))

    def tables(self, t):                             # cos and sin of the angles, [T, H/2] each
        freqs = torch.outer(t.to(torch.float32), self.inv_freq)
        return torch.cos(freqs), torch.sin(freqs)

    def forward(self, x, t):                         # x [B, T, N, H], t [T]
        freqs = torch.outer(t.to(torch.float32), self.inv_freq)
        emb = torch.cat([freqs, freqs], dim=-1)[:, None, :]
        d = x.shape[-1]
        rotated = torch.cat([-x[..., d // 2:], x[..., : d // 2]], dim=-1)
        return x * torch.cos(emb) + rotated * torch.sin(emb)


def group_norm(x, n_groups, eps, scale, bias):
    """flax.nnx.GroupNorm on [B, T, C] (_module.py:118-123): per batch element and group, mean and variance over the
    T positions and the C / n_groups channels of the group (variance as E[x^2] - E[x]^2), then scale and bias."""
    bsz, steps, chans = x.shape
    g = x.reshape(bsz, steps, n_groups, chans // n_groups)
    mean = g.mean(dim=(1, 3), keepdim=True)
    var = torch.clamp((g * g).mean(dim=(1, 3), keepdim=True) - mean * mean, min=0.0)
    out = ((g - mean) * torch.rsqrt(var + eps)).reshape(bsz, steps, chans)
    return out * scale + bias


class TimeMix(torch.nn.Module):                      # _module.py:92-225
    def __init__(self, cfg, gen, device, first_layer):
        super().__init__()
        c, blk = cfg.hidden_size, cfg.blksize
        self.cfg, self.first_layer = cfg, first_layer
        self.n_head, self.head_dim = c // cfg.head_dim, cfg.head_dim
        self.mu = torch.nn.Parameter(_lecun(6, (6, c), gen, device))
        grid = (blk, blk)
        self.w_key, self.w_value = Linear(c, c, grid, gen, device), Linear(c, c, grid, gen, device)
        self.w_output, self.w_receptance = Linear(c, c, grid, gen, device), Linear(c, c, grid, gen, device)
        self.gate_lora, self.decay_lora = LowRankFFN(c, cfg.lora_rank, blk, gen, device), LowRankFFN(c, cfg.lora_rank, blk, gen, device)
        self.iclr_lora = LowRankFFN(c, cfg.lora_rank, blk, gen, device)
        if not first_layer:
            self.nu_lora = LowRankFFN(c, cfg.lora_rank, blk, gen, device)
        self.iclr_mix_amt = torch.nn.Parameter(_lecun(1, (1, c), gen, device))
        self.removal_key_multiplier = torch.nn.Parameter(_lecun(1, (1, c), gen, device))
        self.bonus_multiplier = torch.nn.Parameter(_lecun(1, (1, c), gen, device))
        self.gn_scale = torch.nn.Parameter(torch.ones(c, device=device))
        self.gn_bias = torch.nn.Parameter(torch.zeros(c, device=device))
        self.rotary = RotaryEmbedding(cfg, device)

    def forward(self, x, v_prime_0, t_positions, tm_state, wkv_state):
        bsz, steps, c = x.shape
        n, h, blk = self.n_head, self.head_dim, self.cfg.blksize
        mu = read_param(self.mu, (1, blk))
        if self.cfg.fused_glue and can_quantize_mixes(x, torch.is_grad_enabled()):
            # every mix only feeds linears: they leave the lerp kernel as fp8 triples (the three that feed a (128,128)
            # kernel also in the token-major form its wgrad wants) and are never written as f32
            x_r, x_d, x_k, x_v, x_i, x_g = token_shift_lerp_quantized(x, tm_state, mu, (0, 2, 3) if torch.is_grad_enabled() else ())
        elif self.cfg.fused_glue:
            x_r, x_d, x_k, x_v, x_i, x_g = token_shift_lerp(x, tm_state, mu)
        else:
            x_shifted = torch.cat([tm_state, x[:, :-1, :]], dim=1)
            _x, _xs = x.to(torch.float32), x_shifted.to(torch.float32)
            x_r, x_d, x_k, x_v, x_i, x_g = (lerp(_x, _xs, mu[j]) for j in range(6))
        tm_state = x[:, -1:, :]
        r = self.w_receptance(x_r)
        d = self.decay_lora(x_d)
        k = self.w_key(x_k)
        v_prime = self.w_value(x_v)
        gate = self.gate_lora(x_g)
        iclr = self.iclr_lora(x_i)
        rk_mult = read_param(self.removal_key_multiplier, (1, blk))
        mix_amt = read_param(self.iclr_mix_amt, (1, blk))
        if self.cfg.fused_glue:
            cos_tab, sin_tab = self.rotary.tables(t_positions)
            nu_raw = None if self.first_layer else self.nu_lora(x_v)
            decay, iclr, removal_k, replacement_k, v, r, k = wkv_prepare(
                r, k, d, iclr, v_prime, None if self.first_layer else v_prime_0, nu_raw, cos_tab, sin_tab, rk_mult, mix_amt, n)
            if self.first_layer:
                v_prime_0 = v
        else:
            iclr = torch.sigmoid(iclr)
            k = self.rotary(k.to(torch.float32).reshape(bsz, steps, n, h), t_positions).reshape(bsz, steps, c)
            r = self.rotary(r.to(torch.float32).reshape(bsz, steps, n, h), t_positions).reshape(bsz, steps, c)
            if self.first_layer:
                v = v_prime_0 = v_prime.to(torch.float32)
            else:
                nu = torch.sigmoid(self.nu_lora(x_v)).to(torch.float32)
                v = lerp(v_prime.to(torch.float32), v_prime_0.to(torch.float32), nu)
            decay = torch.exp(-torch.exp(d))
            removal_k = normalized((k * rk_mult).reshape(bsz, steps, n, h), dim=-1).reshape(bsz, steps, c)
            iclr = iclr.to(torch.float32)
            replacement_k = lerp(k, k * iclr, mix_amt)
        wkv_state, out = wkv_state_scan(wkv_state, decay, iclr, removal_k, replacement_k, v, r, n)
        bonus_mult = read_param(self.bonus_multiplier, (1, blk))
        if self.cfg.fused_glue:
            out = wkv_finish(out, r, k, v, gate, self.gn_scale, self.gn_bias, bonus_mult, n * 1e-5, n)
        else:
            out = group_norm(out, n, n * 1e-5, self.gn_scale, self.gn_bias)
            bonus = torch.sum(r * k * bonus_mult, dim=-1, keepdim=True) * v
            out = (out + bonus) * gate.to(torch.float32)
        return self.w_output(out), v, tm_state, wkv_state


class ChannelMix(torch.nn.Module):                   # _module.py:228-258
    def __init__(self, cfg, gen, device):
        super().__init__()
        grid = (cfg.blksize, cfg.blksize)
        self.blk, self.fused_glue = cfg.blksize, cfg.fused_glue
        self.w_k = Linear(cfg.hidden_size, cfg.intermediate_size, grid, gen, device)
        self.w_v = Linear(cfg.intermediate_size, cfg.hidden_size, grid, gen, device)
        self.mu_x = torch.nn.Parameter(_lecun(1, (1, cfg.hidden_size), gen, device))

    def forward(self, x, cm_state):
        mu_x = read_param(self.mu_x, (1, self.blk))
        if self.fused_glue and can_quantize_mixes(x, torch.is_grad_enabled()):
            x_k = token_shift_lerp_quantized(x, cm_state, mu_x, (0,) if torch.is_grad_enabled() else ())[0]
        elif self.fused_glue:
            x_k = token_shift_lerp(x, cm_state, mu_x)[0]
        else:
            x_shifted = torch.cat([cm_state, x[:, :-1, :]], dim=1)
            x_k = lerp(x.to(torch.float32), x_shifted.to(torch.float32), mu_x)
        cm_state = x[:, -1:, :]
        if self.fused_glue and not torch.is_grad_enabled() and x.is_cuda and self.w_k.kernel.shape[1] % 1024 == 0 and self.w_k.tgrid[1] == 128:
            # no backward pass follows (the first pass of a recomputed block): the first product's re-quantization, relu^2 and
            # the second Linear's input quantization are one pass over the f32 product, and k is never written
            y = self.w_k(x_k, raw=True)
            k = QuantizedMix(y.new_zeros(1).expand(y.shape), _ops.relu2_requantize_impl(y), None)
            return self.w_v(k), cm_state
        k = self.w_k(x_k).to(torch.float32)
        if self.fused_glue and torch.is_grad_enabled() and can_quantize_relu2(k) and self.w_v.tgrid == (128, 128):
            k = relu2_quantized(k)       # relu^2 as the prologue of w_v's two input quantizers
        else:
            k = relu2(k) if self.fused_glue else torch.relu(k) ** 2
        return self.w_v(k), cm_state


class RWKVBlock(torch.nn.Module):                    # _module.py:286-317
    def __init__(self, cfg, gen, device, first_layer):
        super().__init__()
        self.tm = TimeMix(cfg, gen, device, first_layer)
        self.cm = ChannelMix(cfg, gen, device)
        self.pre_rmsnorm = RMSNorm(cfg.hidden_size, cfg.blksize, cfg.rmsnorm_epsilon, device, cfg.fused_glue)
        self.post_rmsnorm = RMSNorm(cfg.hidden_size, cfg.blksize, cfg.rmsnorm_epsilon, device, cfg.fused_glue)

    def forward(self, x, v_0, t_positions, tm_state, cm_state, wkv_state):
        x = self.pre_rmsnorm(x)
        dx, v_0, tm_state, wkv_state = self.tm(x, v_0, t_positions, tm_state, wkv_state)
        x = x + dx
        x = self.post_rmsnorm(x)
        dx, cm_state = self.cm(x, cm_state)
        return x + dx, v_0, tm_state, cm_state, wkv_state


class _RematBlock(torch.autograd.Function):
    """A block whose activations are recomputed in the backward pass (the reference's nnx.remat, _model.py:26-30).
    Forward: the block under no_grad from zero states, so none of its layers keeps anything for a backward pass (no X^T
    quantization, no scan checkpoints); only the block's inputs are kept.  Backward: the block again with gradients
    enabled, then its own backward pass; the parameters' gradients accumulate there, the inputs' are returned."""

    @staticmethod
    def forward(ctx, blk, t_positions, zero_state, x, v_0):
        ctx.blk, ctx.t_positions, ctx.zero_state = blk, t_positions, zero_state
        ctx.set_materialize_grads(False)
        ctx.save_for_backward(x, v_0)
        with torch.no_grad():
            y, v, _, _, _ = blk(x, v_0, t_positions, zero_state, zero_state, None)
        return y, v

    @staticmethod
    def backward(ctx, g_y, g_v):
        x, v_0 = ctx.saved_tensors
        x_in = x.detach().requires_grad_(True)
        v_in = v_0.detach().requires_grad_(True) if v_0 is not None else None
        with torch.enable_grad():
            y, v, _, _, _ = ctx.blk(x_in, v_in, ctx.t_positions, ctx.zero_state, ctx.zero_state, None)
        outs = [(y, g_y), (v, g_v)]
        torch.autograd.backward([o for o, g in outs if g is not None], [g for _, g in outs if g is not None])
        return None, None, None, x_in.grad, v_in.grad if v_in is not None else None


class PratchyaCausalLM(torch.nn.Module):
    """PratchyaModel + lm_head + loss, _model.py:10-96 and _utils.py:7-13, from a zero state (`init_state`,
    _config.py:41-52).  `remat=True` recomputes each block in the backward pass, as the reference's nnx.remat does;
    `remat=n` (an int) recomputes the first n blocks only and keeps the activations of the others, for a device whose
    memory holds them (loss and gradients are the same bits for every n: all kernels are deterministic)."""

    def __init__(self, cfg: PratchyaConfig, *, seed: int = 42, device="cuda", remat: bool | int = True):
        super().__init__()
        gen = torch.Generator(device=device).manual_seed(seed)
        self.cfg = cfg
        self.remat = (cfg.n_layers if remat else 0) if isinstance(remat, bool) else max(0, min(int(remat), cfg.n_layers))
        self.embedding = torch.nn.Parameter(torch.randn(cfg.vocab_size, cfg.hidden_size, generator=gen, device=device) / math.sqrt(cfg.hidden_size))
        self.blocks = torch.nn.ModuleList([RWKVBlock(cfg, gen, device, first_layer=i == 0) for i in range(cfg.n_layers)])
        self.pre_rmsnorm = RMSNorm(cfg.hidden_size, cfg.blksize, cfg.rmsnorm_epsilon, device, cfg.fused_glue)
        self.final_rmsnorm = RMSNorm(cfg.hidden_size, cfg.blksize, cfg.rmsnorm_epsilon, device, cfg.fused_glue)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, (cfg.blksize, 1), gen, device)

    def embed(self, input_ids):                      # EmbeddingScaled, _module.py:21-37
        rows = self.embedding[input_ids]             # the rows of a (1,blk)-quantized table quantize as the table does: row-local super-groups
        return read_param(rows, (1, self.cfg.blksize)) * math.sqrt(self.cfg.hidden_size)

    def forward(self, input_ids, label=None, keep_logits=True):
        """(logits, loss).  `keep_logits=False` (with labels, fused kernels): the logits are not returned and the loss's
        backward pass writes their cotangent over them, for a training step that only wants the loss."""
        cfg = self.cfg
        bsz, steps = input_ids.shape
        dev = input_ids.device
        t_positions = torch.arange(steps, device=dev, dtype=torch.int32)
        x = self.pre_rmsnorm(self.embed(input_ids))
        v = None
        zeros_c = torch.zeros(bsz, 1, cfg.hidden_size, device=dev)
        for i, blk in enumerate(self.blocks):
            if i < self.remat and torch.is_grad_enabled():
                x, v = _RematBlock.apply(blk, t_positions, zeros_c, x, v)
            else:
                x, v, _, _, _ = blk(x, v, t_positions, zeros_c, zeros_c, None)
        x = self.final_rmsnorm(x)
        logits = self.lm_head(x)
        loss = None
        if label is not None:
            if cfg.fused_glue:
                loss = fused_cross_entropy(logits, label, reuse_logits=not keep_logits)
                if not keep_logits:
                    logits = None
            else:
                loss = smoothed_cross_entropy(logits, label)
        return logits, loss


def smoothed_cross_entropy(logits, labels, alpha: float = 0.1):
    """compute_loss, _utils.py:7-13, on logits [B, T, V] and labels [B, T]: position t predicts label t+1 (the caller of
    the reference passes logits[:, :-1] and label[:, 1:]); one-hot labels smoothed by alpha (optax.smooth_labels),
    softmax cross entropy in f32, mean over batch and the T-1 positions.  Everything runs on the whole contiguous
    array and the last position gets weight zero, which avoids strided copies of the logits and of their gradient."""
    bsz, steps, _ = logits.shape
    logp = torch.log_softmax(logits.to(torch.float32), dim=-1)
    target = torch.cat([labels[:, 1:], labels[:, :1]], dim=1).to(torch.int64)        # the last column is a placeholder
    nll = -logp.gather(-1, target.unsqueeze(-1)).squeeze(-1)
    uniform = -logp.mean(dim=-1)
    per_position = (1.0 - alpha) * nll + alpha * uniform
    weight = torch.ones(steps, device=logits.device, dtype=torch.float32)
    weight[-1] = 0.0
    return (per_position * weight).sum() / (bsz * (steps - 1))
