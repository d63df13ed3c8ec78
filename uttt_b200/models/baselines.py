"""Baseline language models that share the trainer, the sliding-window attention kernel and the MLP.

* ``transformer``: full-attention or sliding-window Transformer (the reference uses fla's built-in model).
* ``*_swa`` mixers: a bounded-state token mixer in parallel with a sliding-window attention branch computed
  from the same q/k/v projections with a learned affine rescale and rotary
  (uttt_llm/flame/custom_models/fla_window_mix_utils.py:68-133; deltanet_swa/layer_deltanet_swa.py:20-186).
  The mixers are plain PyTorch chunked recurrences: delta rule, gated delta rule, per-channel gated delta rule
  (KDA), Mamba-2 style scalar-decay state space duality, and a mixture of delta-rule memories (MoM).  They
  are baselines, not tuned kernels.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .common import GatedMLP, RMSNorm, SlidingWindowAttention, TokenEmbedding, init_linear_weights
from .uttt_moe import UTTTMoEForCausalLM


class TransformerBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        d = config.hidden_size
        self.attn_norm = RMSNorm(d, eps=config.norm_eps)
        self.attn = SlidingWindowAttention(config, layer_idx)
        self.mlp_norm = RMSNorm(d, eps=config.norm_eps)
        self.mlp = GatedMLP(d, config.mlp_intermediate_size)

    def forward(self, h):
        o = self.attn(self.attn_norm(h), None, None, 0)[0]
        h = h + o
        return h + self.mlp(self.mlp_norm(h))


def chunked_delta_rule(q, k, v, beta, decay=None, chunk: int = 64):
    """Delta-rule memory S_t = a_t S_{t-1} + beta_t k_t (v_t - a_t S_{t-1}^T k_t)^T, read o_t = S_t^T q_t.

    q, k: [b, h, l, dk]; v: [b, h, l, dv]; beta: [b, h, l]; decay a_t in (0, 1]: [b, h, l] or [b, h, l, dk] (per
    key channel) or None.  The state is carried exactly across chunks; inside a chunk the recurrence is stepped
    token by token (a reference implementation, O(l) sequential steps of small einsums).
    """
    b, h, l, dk = k.shape
    dv = v.shape[-1]
    s = q.new_zeros(b, h, dk, dv, dtype=torch.float32)
    outs = []
    qf, kf, vf, bf = q.float(), k.float(), v.float(), beta.float()
    for t in range(l):
        if decay is not None:
            a = decay[:, :, t].float()
            s = s * (a.unsqueeze(-1) if a.dim() == 3 else a.view(b, h, 1, 1))
        kt, vt = kf[:, :, t], vf[:, :, t]
        pred = torch.einsum("bhkv,bhk->bhv", s, kt)
        s = s + torch.einsum("bhk,bhv->bhkv", kt * bf[:, :, t].unsqueeze(-1), vt - pred)
        outs.append(torch.einsum("bhkv,bhk->bhv", s, qf[:, :, t]))
    return torch.stack(outs, dim=2).to(q.dtype)


def chunked_scalar_decay_ssm(q, k, v, log_decay, chunk: int = 64):
    """Mamba-2 style SSD: S_t = exp(g_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, evaluated chunk by chunk with the
    quadratic intra-chunk form and a carried inter-chunk state.  q,k [b,h,l,n]; v [b,h,l,p]; log_decay [b,h,l] <= 0."""
    b, h, l, n = k.shape
    p = v.shape[-1]
    s = q.new_zeros(b, h, n, p, dtype=torch.float32)
    outs = []
    for c0 in range(0, l, chunk):
        qc, kc, vc = q[:, :, c0:c0 + chunk].float(), k[:, :, c0:c0 + chunk].float(), v[:, :, c0:c0 + chunk].float()
        g = log_decay[:, :, c0:c0 + chunk].float().cumsum(-1)                    # [b,h,c]
        w = torch.exp(g.unsqueeze(-1) - g.unsqueeze(-2))                          # decay from j to i
        w = torch.tril(w)
        intra = torch.einsum("bhin,bhjn->bhij", qc, kc) * w
        o = torch.einsum("bhij,bhjp->bhip", intra, vc) + torch.einsum("bhin,bhnp->bhip", qc * torch.exp(g).unsqueeze(-1), s)
        tail = torch.exp(g[:, :, -1:].unsqueeze(-1) - g.unsqueeze(-1))            # decay from j to the chunk end
        s = s * torch.exp(g[:, :, -1]).view(b, h, 1, 1) + torch.einsum("bhjn,bhjp->bhnp", kc * tail.squeeze(-1).unsqueeze(-1), vc)
        outs.append(o)
    return torch.cat(outs, dim=2).to(q.dtype)


class SWAMixerLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        d = config.hidden_size
        self.config = config
        self.mixer = config.mixer
        self.head_dim = config.mixer_head_dim
        self.heads = config.mixer_num_heads or d // self.head_dim
        self.attn_head_dim = config.head_dim
        self.window = config.window_size
        self.theta = float(config.rope_theta or 10000.0)
        self.q_proj = nn.Linear(d, d, bias=False)
        self.k_proj = nn.Linear(d, d, bias=False)
        self.v_proj = nn.Linear(d, d, bias=False)
        self.b_proj = nn.Linear(d, self.heads, bias=False)
        self.g_proj = nn.Linear(d, self.heads if self.mixer != "kda" else d, bias=True) \
            if self.mixer in ("gated_deltanet", "kda", "mamba2") else None
        if self.mixer == "mom":
            self.mem_router = nn.Linear(d, config.num_memories, bias=False)
        self.qk_scale = nn.Parameter(torch.ones(d, 2))
        self.qk_offset = nn.Parameter(torch.zeros(d, 2))
        self.o_norm = RMSNorm(self.head_dim, eps=config.norm_eps)
        self.o_proj = nn.Linear(d, d, bias=False)

    def _mix(self, x, q, k, v):
        b, l, d = x.shape
        h, hd = self.heads, self.head_dim
        qh = F.normalize(F.silu(q).view(b, l, h, hd), dim=-1).transpose(1, 2)
        kh = F.normalize(F.silu(k).view(b, l, h, hd), dim=-1).transpose(1, 2)
        vh = F.silu(v).view(b, l, h, hd).transpose(1, 2)
        beta = torch.sigmoid(self.b_proj(x)).transpose(1, 2)
        if self.mixer == "deltanet":
            return chunked_delta_rule(qh, kh, vh, beta)
        if self.mixer == "gated_deltanet":
            a = torch.exp(-F.softplus(self.g_proj(x))).transpose(1, 2)
            return chunked_delta_rule(qh, kh, vh, beta, a)
        if self.mixer == "kda":
            a = torch.exp(-F.softplus(self.g_proj(x))).view(b, l, h, hd).transpose(1, 2)
            return chunked_delta_rule(qh, kh, vh, beta, a)
        if self.mixer == "mamba2":
            # beta plays the role of the input step size (dt) on the written value
            return chunked_scalar_decay_ssm(qh, kh, vh * beta.unsqueeze(-1).to(vh.dtype),
                                            -F.softplus(self.g_proj(x)).transpose(1, 2))
        if self.mixer == "mom":
            cfg = self.config
            probs = torch.softmax(self.mem_router(x).float(), dim=-1)
            top = probs.topk(cfg.topk_memories, dim=-1)
            gate = torch.zeros_like(probs).scatter(-1, top.indices, top.values)
            gate = gate / gate.sum(-1, keepdim=True).clamp_min(1e-9)
            out = 0
            for m in range(cfg.num_memories):
                gm = gate[..., m].unsqueeze(1)                                    # [b,1,l]
                out = out + chunked_delta_rule(qh, kh, vh, beta * (gm > 0)) * gm.unsqueeze(-1).to(vh.dtype)
            return out
        raise ValueError(f"unknown mixer {self.mixer!r}")

    def forward(self, x):
        b, l, d = x.shape
        q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        mix = self._mix(x, q, k, v)
        mix = self.o_norm(mix.transpose(1, 2).reshape(b, l, self.heads, self.head_dim)).reshape(b, l, d)
        ah = d // self.attn_head_dim
        qa = (q * self.qk_scale[:, 0] + self.qk_offset[:, 0]).view(b, l, ah, self.attn_head_dim)
        ka = (k * self.qk_scale[:, 1] + self.qk_offset[:, 1]).view(b, l, ah, self.attn_head_dim)
        qa, ka = ops.rope(qa, 0, self.theta), ops.rope(ka, 0, self.theta)
        att = ops.swa_attention(qa, ka, v.view(b, l, ah, self.attn_head_dim), self.window, causal=True)
        return self.o_proj(mix + att.reshape(b, l, d).to(mix.dtype))


class SWAMixerBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        d = config.hidden_size
        self.attn_norm = RMSNorm(d, eps=config.norm_eps)
        self.attn = SWAMixerLayer(config, layer_idx)
        self.mlp_norm = RMSNorm(d, eps=config.norm_eps)
        self.mlp = GatedMLP(d, config.mlp_intermediate_size)

    def forward(self, h):
        h = h + self.attn(self.attn_norm(h))
        return h + self.mlp(self.mlp_norm(h))


class _StackModel(nn.Module):
    block_cls = TransformerBlock

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embeddings = TokenEmbedding(config.vocab_size, config.hidden_size, config.pad_token_id)
        self.layers = nn.ModuleList([self.block_cls(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.activation_checkpoint = True
        init_linear_weights(self, config.initializer_range)

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values: Any = None, use_cache: bool = False):
        from torch.utils.checkpoint import checkpoint
        h = self.embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        for layer in self.layers:
            if self.activation_checkpoint and torch.is_grad_enabled():
                h = checkpoint(layer, h, use_reentrant=False, preserve_rng_state=False)
            else:
                h = layer(h)
        h = self.norm(h)
        return h, h.new_zeros((), dtype=torch.float32), None


class TransformerModel(_StackModel):
    block_cls = TransformerBlock


class SWAMixerModel(_StackModel):
    block_cls = SWAMixerBlock


class TransformerForCausalLM(UTTTMoEForCausalLM):
    model_cls = TransformerModel


class SWAMixerForCausalLM(UTTTMoEForCausalLM):
    model_cls = SWAMixerModel
