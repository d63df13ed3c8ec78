"""Dense fast-weight language models.

* uTTT-Dense: one dense SwiGLU operator per fast-weight head, ``[H, r*D, D]``, shared by the whole
  stack; every layer reads it, and at each chunk boundary the mean (or sum) of all layers' inner
  gradients is written once (uttt_llm/flame/custom_models/uttt_dense/modeling_recurrent_lact.py:
  shared bank ``:919-932``, ``_apply_shared_update`` ``:1109-1240``, ``_aggregate_memory_update``
  ``:1302-1386``).
* TTT-Dense / LaCT: the same operator private to each layer, written by that layer only
  (uttt_llm/flame/custom_models/uttt_moe/ref_base.py:500-660; lact/lact_model/layer_lact_swiglu.py).

Both reuse the grouped tensor-core path of the routed models: a fast-weight head is an "expert"
with deterministic routing (row n of a sequence belongs to head n mod H, combine weight 1), so the
same tile-padded layout, grouped GEMMs and fused write-gradient node serve the dense case.
"""
from __future__ import annotations

import os

from typing import Any, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref
from . import fast_weights as fw
from .common import (GatedMLP, LowRankFastWeight, RMSNorm, SlidingWindowAttention, TokenEmbedding, init_linear_weights, inv_softplus,
                     trim_history)
from .uttt_moe import UTTTMoEForCausalLM


def head_routing(bsz: int, n: int, heads: int, device) -> fw.Routing:
    """Deterministic 'routing' of the dense model: row n -> head n mod H with weight one."""
    idx = (torch.arange(n, device=device) % heads).view(1, n, 1).expand(bsz, n, 1).contiguous()
    plan = ops.build_group_plan(idx, heads)
    ones = torch.ones(bsz * n, 1, device=device, dtype=torch.float32)
    zeros = torch.zeros(bsz, heads, device=device, dtype=torch.float32)
    return fw.Routing(plan, ones, zeros, zeros)


def apply_dense_update(a02, a1, state: fw.PoolState, m_coeff, lr_scale: float, use_muon: bool, slices: int,
                       master_renorm: bool, compute_dtype) -> fw.PoolState:
    """Dense write: momentum on the raw aggregate, Newton-Schulz per square D x D slice (``slices`` = r) or
    per whole matrix (``slices`` = 0), master += delta, fast copy = master rescaled row-wise to the *previous
    fast* row norms (the master itself is renormalised only with ``master_renorm``).

    With slices, a "row" is a row of one D x D slice: for the down matrix ``w1`` [D, r*D] every row is r segments of
    D entries with their own norms (uttt_llm/flame/custom_models/uttt_dense/modeling_recurrent_lact.py:1068-1085,
    1166-1216 renormalise the slices, not the wide matrices)."""
    m02, m1 = state.m02, state.m1
    bsz, h, inter2, d = m02.shape
    inter = inter2 // 2
    src02, src1 = (m02, m1) if master_renorm else (state.w02, state.w1)
    seg = (inter // d) if (slices and slices > 0) else 1       # norm segments per row of w1

    def rows1(t):                                              # [b, h, d, inter] -> [b, h, d, seg, inter / seg]
        return t.reshape(bsz, h, d, seg, inter // seg)
    old02 = src02.float().norm(dim=3, keepdim=True)
    old1 = rows1(src1.float()).norm(dim=4, keepdim=True)
    z02, z1 = state.z02, state.z1
    if z02 is not None and m_coeff is not None:
        a02 = a02 + z02 * m_coeff
        a1 = a1 + z1 * m_coeff
        z02, z1 = a02, a1
    if use_muon:
        if slices and slices > 0:
            r = inter // d
            # w0|w2: [b,h,2,r,d,d] -> independent squares; w1: [b,h,d,r,d] -> [b,h,r,d,d]
            d02 = ops.newton_schulz(a02.reshape(bsz * h * 2 * r, d, d)).reshape(bsz, h, inter2, d)
            s1 = a1.reshape(bsz, h, d, r, d).permute(0, 1, 3, 2, 4).reshape(bsz * h * r, d, d)
            d1 = ops.newton_schulz(s1).reshape(bsz, h, r, d, d).permute(0, 1, 3, 2, 4).reshape(bsz, h, d, inter)
        else:
            d02 = ops.newton_schulz(a02.reshape(bsz * h * 2, inter, d)).reshape(bsz, h, inter2, d)
            d1 = ops.newton_schulz(a1.reshape(bsz * h, d, inter)).reshape(bsz, h, d, inter)
    else:
        d02, d1 = a02, a1
    n02 = m02 + d02.float() * lr_scale
    n1 = m1 + d1.float() * lr_scale
    p02 = n02 / (n02.norm(dim=3, keepdim=True) + 1e-5) * old02
    p1 = (rows1(n1) / (rows1(n1).norm(dim=4, keepdim=True) + 1e-5) * old1).reshape(bsz, h, d, inter)
    if master_renorm:
        n02, n1 = p02, p1
    return fw.PoolState(p02.to(compute_dtype), p1.to(compute_dtype), n02, n1, z02, z1)


class DenseBlock(nn.Module):
    def __init__(self, config, layer_idx: int, private_weights: bool):
        super().__init__()
        self.config = config
        d = config.hidden_size
        self.attn_norm = RMSNorm(d, eps=config.norm_eps)
        self.attn = SlidingWindowAttention(config, layer_idx)
        self.memory = fw.FastWeightMemory(config, layer_idx, momentum_out=config.fw_heads)
        self.memory_norm = RMSNorm(d, eps=config.norm_eps) if config.residual_style == "sequential" else None
        self.to_lr = nn.Linear(d, 3 * config.fw_heads if config.per_head_lr else 3)
        self.base_lr_inv = inv_softplus(config.base_lr)
        self.memory_output_proj = nn.Linear(d, d, bias=False) if config.enable_attention_memory_output_proj else None
        self.mlp_norm = RMSNorm(d, eps=config.norm_eps)
        self.mlp = GatedMLP(d, config.mlp_intermediate_size)
        if private_weights:
            h, dd, ii = config.fw_heads, config.fw_head_dim, config.fw_inter_dim
            if config.w0_w2_low_rank > 0:
                # identity / 2 plus a low-rank product (ttt_dense/modeling_recurrent_lact.py:138-186, 227-244)
                self.memory.w0 = LowRankFastWeight(h, ii, dd, config.w0_w2_low_rank, config.fw_init_gain, True)
                self.memory.w2 = LowRankFastWeight(h, ii, dd, config.w0_w2_low_rank, config.fw_init_gain, True)
            else:
                self.memory.w0 = nn.Parameter(torch.randn(h, ii, dd) / dd ** 0.5)
                self.memory.w2 = nn.Parameter(torch.randn(h, ii, dd) / dd ** 0.5)
            self.memory.w1 = nn.Parameter(torch.randn(h, dd, ii) / ii ** 0.5)

    def private_weights(self):
        """(w0, w1, w2) of a block that owns its fast weights."""
        m = self.memory
        if isinstance(m.w0, LowRankFastWeight):
            return m.w0(), m.w1, m.w2()
        return m.w0, m.w1, m.w2

    def forward(self, h, k_hist, v_hist, w02, w1, offset: int):
        cfg = self.config
        residual = h
        x_in = self.attn_norm(h)
        attn_out, q_flat, k_flat, v_flat, k_rot, v_new = self.attn(x_in, k_hist, v_hist, offset)
        mem = self.memory
        if cfg.residual_style == "sequential":
            h, x_mem = self.memory_norm.add_forward(residual, attn_out)
            residual = h
        else:
            x_mem = x_in
        q_rows = mem.head_rows(mem.prep_query(q_flat, offset))
        routing = head_routing(q_rows.shape[0], q_rows.shape[1], mem.fw_heads, q_rows.device)
        y = fw.pool_read(q_rows, w02, w1, routing)
        mem_out = mem.finish_read(y, x_mem).to(attn_out.dtype)
        mixed = mem_out + attn_out if cfg.residual_style == "parallel" else mem_out
        if self.memory_output_proj is not None:
            mixed = self.memory_output_proj(mixed)
        h, x_mlp_in = self.mlp_norm.add_forward(residual, mixed)
        h = h + self.mlp(x_mlp_in)
        return h, x_in, k_flat, v_flat, k_rot, v_new

    def raw_grad(self, x_in, k_flat, v_flat, w02, w1, offset: int, acc=None):
        mem = self.memory
        b, l, _ = x_in.shape
        lr = F.softplus(self.to_lr(x_in).float() + self.base_lr_inv)
        if lr.shape[-1] == 3:
            lr_rows = lr.unsqueeze(2).expand(b, l, mem.fw_heads, 3).reshape(b, l * mem.fw_heads, 3)
        else:
            lr_rows = lr.reshape(b, l * mem.fw_heads, 3)
        k_rows = mem.head_rows(mem.prep_key(k_flat, offset))
        v_rows = mem.head_rows(mem.prep_value(v_flat))
        routing = head_routing(b, k_rows.shape[1], mem.fw_heads, k_rows.device)
        g02, g1 = fw.pool_raw_grad(k_rows, v_rows, lr_rows, w02, w1, routing, acc=acc)
        m = mem.momentum_coeff(x_in)          # [b, H]
        return g02, g1, m


class DenseFWModel(nn.Module):
    """Backbone of uTTT-Dense (``shared=True``) and TTT-Dense / LaCT (``shared=False``)."""

    shared = True

    def __init__(self, config):
        super().__init__()
        self.config = config
        d = config.hidden_size
        self.embeddings = TokenEmbedding(config.vocab_size, d, config.pad_token_id)
        self.layers = nn.ModuleList([DenseBlock(config, i, private_weights=not self.shared)
                                     for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(d, eps=config.norm_eps)
        self.activation_checkpoint = True
        if self.shared:
            h, dd = config.fw_heads, config.fw_head_dim
            r = int(config.fw_inter_multi)
            rank = config.w0_w2_low_rank
            if rank > 0:
                self.shared_w0_left = nn.Parameter(torch.empty(h, r, dd, rank))
                self.shared_w0_right = nn.Parameter(torch.empty(h, r, rank, dd))
                self.shared_w2_left = nn.Parameter(torch.empty(h, r, dd, rank))
                self.shared_w2_right = nn.Parameter(torch.empty(h, r, rank, dd))
            else:
                self.shared_w0 = nn.Parameter(torch.empty(h, r * dd, dd))
                self.shared_w2 = nn.Parameter(torch.empty(h, r * dd, dd))
            self.shared_w1 = nn.Parameter(torch.empty(h, dd, r * dd))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        cfg = self.config
        init_linear_weights(self, cfg.initializer_range)
        dd, ii = cfg.fw_head_dim, cfg.fw_inter_dim
        for layer in self.layers:
            layer.memory.reset_parameters()
            if not self.shared:
                if isinstance(layer.memory.w0, LowRankFastWeight):
                    layer.memory.w0.reset_parameters()
                    layer.memory.w2.reset_parameters()
                else:
                    nn.init.normal_(layer.memory.w0, std=dd ** -0.5)
                    nn.init.normal_(layer.memory.w2, std=dd ** -0.5)
                nn.init.normal_(layer.memory.w1, std=ii ** -0.5)
        if self.shared:
            if cfg.w0_w2_low_rank > 0:
                g = cfg.fw_init_gain
                for p in (self.shared_w0_left, self.shared_w2_left):
                    nn.init.normal_(p, std=g / cfg.w0_w2_low_rank ** 0.5)
                for p in (self.shared_w0_right, self.shared_w2_right):
                    nn.init.normal_(p, std=g / dd ** 0.5)
            else:
                nn.init.normal_(self.shared_w0, std=dd ** -0.5)
                nn.init.normal_(self.shared_w2, std=dd ** -0.5)
            nn.init.normal_(self.shared_w1, std=ii ** -0.5)

    def compute_dtype(self) -> torch.dtype:
        return self.embeddings.weight.dtype

    def _shared_weights(self):
        cfg = self.config
        if cfg.w0_w2_low_rank > 0:
            eye = 0.5 * torch.eye(cfg.fw_head_dim, device=self.shared_w1.device)
            h = cfg.fw_heads
            w0 = (self.shared_w0_left.float() @ self.shared_w0_right.float() + eye).reshape(h, -1, cfg.fw_head_dim)
            w2 = (self.shared_w2_left.float() @ self.shared_w2_right.float() + eye).reshape(h, -1, cfg.fw_head_dim)
            return w0, self.shared_w1, w2
        return self.shared_w0, self.shared_w1, self.shared_w2

    def init_states(self, bsz: int) -> List[fw.PoolState]:
        cfg = self.config
        dt = self.compute_dtype()
        if self.shared:
            w0, w1, w2 = self._shared_weights()
            return [fw.init_pool_state(w0, w1, w2, bsz, cfg.use_momentum, dt)]
        return [fw.init_pool_state(*l.private_weights(), bsz, cfg.use_momentum, dt)
                for l in self.layers]

    def _ckpt(self, fn, *args):
        from torch.utils.checkpoint import checkpoint
        if self.activation_checkpoint and torch.is_grad_enabled():
            return checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False)
        return fn(*args)

    def _write(self, states, feats, offset):
        cfg = self.config
        mode = getattr(cfg, "memory_update_backward_mode", "full")
        dt = states[0].w02.dtype
        detach_g = mode in ("first_order_state", "stop_state")
        n_layers = len(self.layers)

        def pack(state):
            return [t for t in state.tensors() if t is not None]

        def unpack(vals):
            vals = list(vals)
            return fw.PoolState.from_tensors(vals + [None] * (6 - len(vals)))

        if self.shared:
            flat = [t for f in feats for t in f]

            def _agg(*args):
                f = args[:3 * n_layers]
                s = unpack(args[3 * n_layers:])
                # the sums of the first pass over this region are kept for its recomputation, which then records
                # the writers' nodes without redoing their GEMMs and reductions (as in models/uttt_moe.py)
                store = getattr(self, "_aggregate_store", None)
                kept = None
                if (store is not None and not detach_g and torch.is_grad_enabled()
                        and ops.fw_write_accumulate_skips(s.m02, s.w02)):
                    kept = store.pop(offset, None)
                else:
                    store = None
                if kept is not None:
                    a02, a1 = kept
                else:
                    a02, a1 = torch.zeros_like(s.m02), torch.zeros_like(s.m1)
                stash = None if (detach_g or kept is not None) else ops.write_stash_for(a02)
                ms = []
                for li, layer in enumerate(self.layers):
                    if detach_g:
                        g02, g1, m = layer.raw_grad(f[3 * li], f[3 * li + 1], f[3 * li + 2], s.w02, s.w1, offset)
                        a02, a1 = a02 + g02.detach(), a1 + g1.detach()
                    else:
                        a02, a1, m = layer.raw_grad(f[3 * li], f[3 * li + 1], f[3 * li + 2], s.w02, s.w1, offset,
                                                    acc=(a02, a1, stash, li == n_layers - 1, kept is not None))
                    if m is not None:
                        ms.append(m)
                if store is not None and kept is None:
                    store[offset] = (a02.detach(), a1.detach())
                if getattr(cfg, "uttt_agg_reduce", "mean") == "mean":
                    a02, a1 = a02 / n_layers, a1 / n_layers
                mc = torch.stack(ms).mean(0).view(a02.shape[0], -1, 1, 1) if ms else None
                new = apply_dense_update(a02, a1, s, mc, getattr(cfg, "uttt_agg_lr_scale", 1.0), cfg.use_moun,
                                         int(cfg.fw_inter_multi), getattr(cfg, "uttt_master_renorm", False), dt)
                return tuple(pack(new))

            args = (*flat, *pack(states[0]))
            out = self._ckpt(_agg, *args) if mode != "stop_state" else _agg(*args)
            new = unpack(out)
            return [new.detach() if mode == "stop_state" else new]

        new_states = []
        for li, layer in enumerate(self.layers):
            def _one(x_in, k_flat, v_flat, *st, _layer=layer):
                s = unpack(st)
                g02, g1, m = _layer.raw_grad(x_in, k_flat, v_flat, s.w02, s.w1, offset)
                if detach_g:
                    g02, g1 = g02.detach(), g1.detach()
                mc = None if m is None else m.view(g02.shape[0], -1, 1, 1)
                return tuple(pack(apply_dense_update(g02, g1, s, mc, 1.0, cfg.use_moun, 0, False, dt)))

            args = (*feats[li], *pack(states[li]))
            out = self._ckpt(_one, *args) if mode != "stop_state" else _one(*args)
            new = unpack(out)
            new_states.append(new.detach() if mode == "stop_state" else new)
        return new_states

    def forward(self, input_ids=None, inputs_embeds=None, past_key_values: Any = None, use_cache: bool = False):
        cfg = self.config
        if inputs_embeds is None:
            inputs_embeds = self.embeddings(input_ids)
        bsz, seq_len, _ = inputs_embeds.shape
        chunk = cfg.chunk_size
        states = self.init_states(bsz)
        n_layers = len(self.layers)
        hist = [(None, None)] * n_layers
        keep = self.layers[0].attn.history_len(chunk) if cfg.window_size is not None else None
        outputs = []
        reuse = (self.activation_checkpoint and self.training and torch.is_grad_enabled()
                 and os.environ.get("UTTT_B200_REUSE_ATTENTION", "1") != "0")
        for layer in self.layers:
            layer.attn.reuse_store = {} if reuse else None      # attention outputs kept for the recomputation
        self._aggregate_store = {} if (reuse and getattr(cfg, "memory_update_backward_mode", "full") == "full"
                                       and os.environ.get("UTTT_B200_REUSE_AGGREGATE", "1") != "0") else None
        for start in range(0, seq_len, chunk):
            end = min(start + chunk, seq_len)
            h = inputs_embeds[:, start:end]
            feats = []
            for li, layer in enumerate(self.layers):
                st = states[0] if self.shared else states[li]
                k_hist, v_hist = hist[li]
                h, x_in, k_flat, v_flat, k_rot, v_new = self._ckpt(layer, h, k_hist, v_hist, st.w02, st.w1, start)
                hist[li] = trim_history(k_hist, v_hist, k_rot, v_new, keep)
                feats.append((x_in, k_flat, v_flat))
            outputs.append(h)
            if end < seq_len:
                states = self._write(states, feats, start)
        hidden = self.norm(torch.cat(outputs, dim=1))
        return hidden, hidden.new_zeros((), dtype=torch.float32), None


class UTTTDenseModel(DenseFWModel):
    shared = True


class TTTDenseModel(DenseFWModel):
    shared = False


class UTTTDenseForCausalLM(UTTTMoEForCausalLM):
    model_cls = UTTTDenseModel


class TTTDenseForCausalLM(UTTTMoEForCausalLM):
    model_cls = TTTDenseModel


class LaCTForCausalLM(TTTDenseForCausalLM):
    """Published LaCT baseline: layer-private large-chunk TTT with SwiGLU fast weights.

    The parameters map one to one onto the reference's ``LaCTForCausalLM`` (lact/lact_model/layer_lact_swiglu.py), which
    keeps them all under ``layers.N.attn`` with a fused ``qkv`` projection.  :meth:`load_state_dict` accepts that
    layout (detected by its ``attn.qkv.weight`` keys) and :meth:`reference_state_dict` writes it."""

    _TO_MEMORY = ("momentum_proj.", "qk_scale", "qk_offset", "ttt_norm.", "ttt_scale_proj.", "w0", "w1", "w2")

    @classmethod
    def from_reference_keys(cls, sd):
        out = {}
        for k, v in sd.items():
            if ".attn." not in k:
                out[k] = v
                continue
            head, tail = k.split(".attn.", 1)
            if tail == "qkv.weight":
                q, kk, vv = v.chunk(3, dim=0)
                out[f"{head}.attn.q_proj.weight"], out[f"{head}.attn.k_proj.weight"] = q, kk
                out[f"{head}.attn.v_proj.weight"] = vv
            elif tail.startswith("o_proj."):
                out[f"{head}.memory_output_proj.{tail[7:]}"] = v
            elif tail.startswith("lr_proj."):
                out[f"{head}.to_lr.{tail[8:]}"] = v
            elif tail.startswith(cls._TO_MEMORY):
                out[f"{head}.memory.{tail}"] = v
            else:
                out[k] = v
        return out

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        if any(k.endswith(".attn.qkv.weight") for k in state_dict):
            state_dict = self.from_reference_keys(state_dict)
        return super().load_state_dict(state_dict, strict=strict, assign=assign)

    def reference_state_dict(self):
        sd, out = self.state_dict(), {}
        for k, v in sd.items():
            if k.endswith(".attn.q_proj.weight"):
                head = k[:-len(".attn.q_proj.weight")]
                out[f"{head}.attn.qkv.weight"] = torch.cat([v, sd[f"{head}.attn.k_proj.weight"],
                                                            sd[f"{head}.attn.v_proj.weight"]], dim=0)
            elif k.endswith((".attn.k_proj.weight", ".attn.v_proj.weight")):
                continue
            elif ".memory_output_proj." in k:
                out[k.replace(".memory_output_proj.", ".attn.o_proj.")] = v
            elif ".to_lr." in k:
                out[k.replace(".to_lr.", ".attn.lr_proj.")] = v
            elif ".memory." in k:
                out[k.replace(".memory.", ".attn.")] = v
            else:
                out[k] = v
        return out
