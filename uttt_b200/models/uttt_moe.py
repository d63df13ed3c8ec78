"""uTTT-MoE / TTT-MoE language model: sliding-window attention plus a routed pool of SwiGLU
fast-weight experts that is read by every layer and written once per chunk.

Behavioural reference: uttt_llm/flame/custom_models/uttt_moe/modeling_recurrent_lact.py
(block ``:929-1017``, chunk loop ``:3490-3554``, aggregate write ``:2381-2546``, update rule
``:754-825``, loss-free balancing ``:1593-1712``, cross-layer cut ``:1379-1529``) and, for the
layer-local pools, uttt_llm/flame/custom_models/ttt_moe_lb/modeling_recurrent_lact.py:125-698.

Design differences (same math):
* chunk-major schedule with one recompute region per (chunk, layer) and one per chunk-boundary
  write, but key/value history is carried as tensors (last ``window-1`` positions) instead of a
  full-length in-place module buffer, and keys/values are projected once per chunk;
* gate and up fast weights stay fused (``[B, E, 2I, D]``) for the whole sequence;
* routing builds a tile-padded expert-major layout on the device without host syncs.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..config import LMConfig
from . import fast_weights as fw
from ..utils.trace import trace_range
from .common import (GatedMLP, LowRankFastWeight, RMSNorm, SlidingWindowAttention, TokenEmbedding, init_linear_weights,
                     inv_softplus, trim_history)


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    ce_loss: Optional[torch.Tensor] = None
    lb_loss: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    moe_stats: Optional[Dict[str, Any]] = None
    past_key_values: Any = None


class MoEBlock(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        d = config.hidden_size
        self.attn_norm = RMSNorm(d, eps=config.norm_eps)
        self.attn = SlidingWindowAttention(config, layer_idx)
        if config.use_memory_block:
            self.memory_norm = RMSNorm(d, eps=config.norm_eps) if config.residual_style == "sequential" else None
            self.memory = fw.FastWeightMemory(config, layer_idx, momentum_out=1)
            self.to_lr = nn.Linear(d, 3 * config.fw_heads if config.per_head_lr else 3)
            self.base_lr_inv = inv_softplus(config.base_lr)
        else:
            self.memory_norm = None
            self.memory = None
        self.memory_output_proj = nn.Linear(d, d, bias=False) if config.enable_attention_memory_output_proj else None
        self.mlp_norm = RMSNorm(d, eps=config.norm_eps)
        self.mlp = GatedMLP(d, config.mlp_intermediate_size)
        self.return_memory_input = False   # set by the model when a write source other than the default is configured
        self.ep = None            # expert-parallel handle, set by the model
        self.write_recomputed = False   # set by the model: the chunk write of this layer runs twice (recomputation)
        self.route_stats = None   # (reads, writes) RouteStats while the model collects pool statistics

    def _reuse(self, offset: int, what: str):
        """(store, key) under which a routed call of this layer keeps its result for the recomputation, or None."""
        store = self.attn.reuse_store
        if store is None or self.ep is not None or os.environ.get("UTTT_B200_REUSE_ROUTING", "1") == "0":
            return None
        return (store, (offset, what))

    # -------------------------------------------------------------------------- read
    def forward(self, h, k_hist, v_hist, w02, w1, router, bias, offset: int):
        """One (chunk, layer) step.  Returns tensors only (it runs under activation recompute)."""
        cfg = self.config
        residual = h
        x_attn_in = self.attn_norm(h)
        attn_out, q_flat, k_flat, v_flat, k_rot, v_new = self.attn(x_attn_in, k_hist, v_hist, offset)
        lb_probs = lb_counts = None
        x_mem_in = x_attn_in
        if self.memory is not None:
            if cfg.residual_style == "sequential":
                h, x_mem_in = self.memory_norm.add_forward(residual, attn_out)
                residual = h
            else:
                x_mem_in = x_attn_in
            mem = self.memory
            # query source (ref_base.py:914-919): the attention's own query, the attention's q projection of the
            # memory input, or the memory's own projection
            if getattr(cfg, "memory_kv_mode", "reuse_kv") == "reuse_kv":
                q_src = q_flat
            elif cfg.memory_kv_proj == "reuse_attn_kv_proj":
                q_src = ops.linear(x_mem_in, self.attn.q_proj.weight, self.attn.q_proj.bias)
            else:
                q_src = ops.linear(x_mem_in, mem.to_q.weight)
            q_rows = mem.head_rows(mem.prep_query(q_src, offset))
            routing = fw.route_rows(q_rows, router, bias, cfg, getattr(cfg, "memory_bias_in_logits", False), self.ep,
                                    reuse=self._reuse(offset, "read"))
            if self.route_stats is not None:          # set by the model for the first pass of a statistics step
                self.route_stats[0].add(q_rows, router, routing.weights)
            y = fw.pool_read(q_rows, w02, w1, routing)
            mem_out = mem.finish_read(y, x_mem_in).to(attn_out.dtype)
            lb_probs, lb_counts = routing.prob_sum, routing.counts
            mixed = mem_out + attn_out if cfg.residual_style == "parallel" else mem_out
        else:
            mixed = attn_out
        if self.memory_output_proj is not None:
            mixed = ops.linear(mixed, self.memory_output_proj.weight)
        h, x_mlp_in = self.mlp_norm.add_forward(residual, mixed)
        h = h + self.mlp(x_mlp_in)
        if lb_probs is None:
            lb_probs = h.new_zeros((h.shape[0], 1), dtype=torch.float32)
            lb_counts = lb_probs
        if self.return_memory_input:
            # only for the write sources that read it (see UTTTMoEModel.compose_write_inputs)
            return h, x_attn_in, k_flat, v_flat, k_rot, v_new, lb_probs, lb_counts, x_mem_in
        return h, x_attn_in, k_flat, v_flat, k_rot, v_new, lb_probs, lb_counts

    # -------------------------------------------------------------------------- write
    def raw_grad(self, x_in, k_flat, v_flat, w02, w1, router, bias, offset: int, acc=None):
        """This layer's lr-weighted inner gradient on the shared bank (added to ``acc`` when given),
        plus momentum gate and lb sums."""
        cfg = self.config
        mem = self.memory
        b, l, _ = x_in.shape
        lr = F.softplus(self.to_lr(x_in).float() + self.base_lr_inv)          # [b, l, 3h] or [b, l, 3]
        if lr.shape[-1] == 3:
            lr_rows = lr.unsqueeze(2).expand(b, l, mem.fw_heads, 3).reshape(b, l * mem.fw_heads, 3)
        else:
            lr_rows = lr.reshape(b, l * mem.fw_heads, 3)
        k_rows = mem.head_rows(mem.prep_key(k_flat, offset))
        v_rows = mem.head_rows(mem.prep_value(v_flat))
        route_in = v_rows if cfg.memory_router_from_v else k_rows
        routing = fw.route_rows(route_in, router, bias, cfg, getattr(cfg, "memory_bias_in_logits", False), self.ep,
                                reuse=self._reuse(offset, "write") if self.write_recomputed else None)
        if self.route_stats is not None:
            self.route_stats[1].add(route_in, router, routing.weights)
        g02, g1 = fw.pool_raw_grad(k_rows, v_rows, lr_rows, w02, w1, routing, acc=acc)
        m = mem.momentum_coeff(x_in)
        return g02, g1, m, routing.prob_sum, routing.counts


def memory_compose_modes(cfg) -> Tuple[str, str]:
    """Where the keys and the values of the write come from (ref_base.py:78-147): ``reuse`` the attention's own
    pre-rotary k / v, ``attn-proj`` = the attention's k / v projection applied to a feature, ``shared`` = one
    model-level projection, ``ttt-proj`` = the memory's own projection."""
    explicit_k = getattr(cfg, "memory_k_compose_mode", None)
    explicit_v = getattr(cfg, "memory_v_compose_mode", None)
    if explicit_k is None and explicit_v is None:
        if getattr(cfg, "memory_perlayer_k_share_v", False):
            return "attn-proj", "shared"
        if getattr(cfg, "memory_perlayer_k_reuse_v", False):
            return "attn-proj", "reuse"
        if getattr(cfg, "memory_shared_kv_cache", False):
            return "shared", "shared"
        if getattr(cfg, "memory_reuse_kv_cache", False):
            return "reuse", "reuse"
    if getattr(cfg, "memory_kv_mode", "reuse_kv") == "reuse_kv":
        base = "reuse"
    else:
        table = {"reuse_attn_kv_proj": "attn-proj", "model_kv_proj": "shared", "ttt_kv_proj": "ttt-proj"}
        if cfg.memory_kv_proj not in table:
            raise ValueError(f"Invalid memory_kv_proj: {cfg.memory_kv_proj}")
        base = table[cfg.memory_kv_proj]
    k_mode = v_mode = base
    if getattr(cfg, "memory_v_gap", None) is not None and explicit_v is None:
        v_mode = "attn-proj"          # a gapped value source is normalised and sent through the attention's v projection
    return explicit_k or k_mode, explicit_v or v_mode


class UTTTMoEModel(nn.Module):
    """Backbone.  ``pool_mode='shared'``: one pool for the whole stack (uTTT-MoE);
    ``'per_layer'``: each layer routes within its own pool (TTT-MoE)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        d = config.hidden_size
        self.embeddings = TokenEmbedding(config.vocab_size, d, config.pad_token_id)
        self.layers = nn.ModuleList([MoEBlock(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(d, eps=config.norm_eps)
        self.num_experts = config.memory_num_experts
        self.per_layer_pool = config.memory_pool_mode != "shared"
        write_layers = config.memory_write_layers
        n_layers = config.num_hidden_layers
        if write_layers == "all":
            self.writer_layers = tuple(range(n_layers))
        elif write_layers == "last":
            self.writer_layers = (n_layers - 1,)
        else:
            self.writer_layers = tuple(sorted(int(i) for i in write_layers))
        self.activation_checkpoint = True
        # layers whose (chunk, layer) regions keep their activations instead of recomputing them in backward:
        # trades spare HBM for one forward pass of those layers
        self.keep_activation_layers = frozenset()
        self.ep = None
        if config.use_memory_block:
            self._init_write_sources()
            self._init_pool_parameters()
            self._init_loss_free_buffers()
            if self.per_layer_pool:
                # layer-local pools are kept as one stacked tensor here (one grouped launch serves every layer's
                # state), but a checkpoint holds them under the owning layer, as the reference's does
                self._register_state_dict_hook(UTTTMoEModel._split_pools_for_state_dict)
                self._register_load_state_dict_pre_hook(self._merge_pools_from_state_dict)
        self.reset_parameters()

    # ------------------------------------------------------------------ checkpoint layout of layer-local pools
    # Reference layout (uttt_llm/flame/custom_models/ttt_moe_lb/modeling_recurrent_lact.py:137-158):
    #   layers.{l}.memory.w0 / w2 [E, I, D] (or .w0.w_left [E, I, r], .w0.w_right [E, r, D]), layers.{l}.memory.w1
    #   [E, D, I], layers.{l}.memory.router_proj_weights [1, E, D].
    _POOL_KEYS = (("pool_w0", "w0"), ("pool_w2", "w2"), ("pool_w1", "w1"), ("pool_w0.w_left", "w0.w_left"),
                  ("pool_w0.w_right", "w0.w_right"), ("pool_w2.w_left", "w2.w_left"),
                  ("pool_w2.w_right", "w2.w_right"))

    @staticmethod
    def _split_pools_for_state_dict(module, state_dict, prefix, local_metadata):
        n_layers, e = module.config.num_hidden_layers, module.num_experts
        for ours, theirs in UTTTMoEModel._POOL_KEYS:
            t = state_dict.pop(prefix + ours, None)
            if t is None:
                continue
            for l in range(n_layers):
                state_dict[f"{prefix}layers.{l}.memory.{theirs}"] = t[l * e:(l + 1) * e]
        r = state_dict.pop(prefix + "per_layer_router_proj_weights", None)
        if r is not None:
            for l in range(n_layers):
                state_dict[f"{prefix}layers.{l}.memory.router_proj_weights"] = r[l]
        return state_dict

    def _merge_pools_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys,
                                     error_msgs):
        n_layers = self.config.num_hidden_layers
        for ours, theirs in UTTTMoEModel._POOL_KEYS:
            keys = [f"{prefix}layers.{l}.memory.{theirs}" for l in range(n_layers)]
            if all(k in state_dict for k in keys):
                state_dict[prefix + ours] = torch.cat([state_dict.pop(k) for k in keys], dim=0)
        keys = [f"{prefix}layers.{l}.memory.router_proj_weights" for l in range(n_layers)]
        if all(k in state_dict for k in keys):
            state_dict[prefix + "per_layer_router_proj_weights"] = torch.stack([state_dict.pop(k) for k in keys], dim=0)

    # ------------------------------------------------------------------ parameters
    def _init_write_sources(self) -> None:
        """Sources of the write's keys / values other than the attention's own k / v of the same layer: gapped
        layers, projections of a feature (ref_base.py:1090-1141)."""
        cfg = self.config
        n = cfg.num_hidden_layers
        self.k_mode, self.v_mode = memory_compose_modes(cfg)
        self.k_gap, self.v_gap = getattr(cfg, "memory_k_gap", None), getattr(cfg, "memory_v_gap", None)
        self.k_source = [max(min(i + (self.k_gap or 0), n - 1), 0) for i in range(n)]
        self.v_source = [max(min(i + (self.v_gap or 0), n - 1), 0) for i in range(n)]
        if (getattr(cfg, "memory_kv_mode", "reuse_kv") != "reuse_kv" and cfg.memory_kv_proj == "model_kv_proj"):
            # the query would need the memory's own projection, which only memory_kv_proj="ttt_kv_proj" creates
            # (the reference fails on its first forward with this combination)
            raise ValueError('memory_kv_mode="to_kv" with memory_kv_proj="model_kv_proj" has no query projection; '
                             'use memory_k_compose_mode / memory_v_compose_mode = "shared" with memory_kv_mode='
                             '"reuse_kv"')
        self.write_feature = getattr(cfg, "memory_kv_feature", "x_attn_in")
        if self.write_feature not in ("x_attn_in", "x_memory_in"):
            raise ValueError(f"memory_kv_feature must be 'x_attn_in' or 'x_memory_in', got {self.write_feature!r}")
        self.default_write_source = (self.k_mode == "reuse" and self.v_mode == "reuse" and not self.k_gap
                                     and not self.v_gap)
        d = cfg.hidden_size
        kv_dim = cfg.kv_heads * cfg.head_dim
        self.pre_memory_v_rms_norm = (RMSNorm(d, eps=cfg.norm_eps)
                                      if self.v_gap is not None and self.v_mode in ("attn-proj", "shared") else None)
        self.memory_shared_k_proj = nn.Linear(d, kv_dim, bias=cfg.qkv_bias) if self.k_mode == "shared" else None
        self.memory_shared_v_proj = nn.Linear(d, kv_dim, bias=cfg.qkv_bias) if self.v_mode == "shared" else None
        want_memory_input = (not self.default_write_source or cfg.memory_kv_mode != "reuse_kv"
                             or (self.write_feature == "x_memory_in" and cfg.residual_style == "sequential"))
        for layer in self.layers:
            layer.return_memory_input = bool(want_memory_input)

    def compose_write_inputs(self, caches: List[Dict[str, torch.Tensor]]) -> List[Tuple[torch.Tensor, ...]]:
        """Per layer (feature for learning rates and momentum, keys, values) of this chunk's write, from the layers'
        caches {x_attn_in, x_memory_in, xi_out, attn_k, attn_v} (ref_base.py:1219-1261)."""
        out = []
        for li, layer in enumerate(self.layers):
            ck, cv = caches[self.k_source[li]], caches[self.v_source[li]]
            pre = k_feature = ck[self.write_feature]
            if self.v_gap is not None:
                v_feature = cv["xi_out"]
                if self.pre_memory_v_rms_norm is not None:
                    v_feature = self.pre_memory_v_rms_norm(v_feature)
            else:
                v_feature = cv[self.write_feature]
            ki = self._project_write_source(layer, self.k_mode, "k", k_feature, ck["attn_k"])
            vi = self._project_write_source(layer, self.v_mode, "v", v_feature, cv["attn_v"])
            out.append((pre, ki, vi))
        return out

    def _project_write_source(self, layer, mode: str, which: str, feature, own):
        if mode == "reuse":
            return own
        if mode == "attn-proj":
            proj = layer.attn.k_proj if which == "k" else layer.attn.v_proj
        elif mode == "shared":
            proj = self.memory_shared_k_proj if which == "k" else self.memory_shared_v_proj
        elif mode == "ttt-proj":
            proj = layer.memory.to_k if which == "k" else layer.memory.to_v
        else:
            raise ValueError(f"Invalid memory compose mode: {mode}")
        return self._ckpt(lambda f, _p=proj: ops.linear(f, _p.weight, _p.bias), feature)

    def _init_pool_parameters(self) -> None:
        cfg = self.config
        e, i_dim, d_dim = cfg.memory_num_experts, cfg.fw_inter_dim, cfg.fw_head_dim
        n_pools = cfg.num_hidden_layers if self.per_layer_pool else 1
        heads = e * n_pools
        if cfg.w0_w2_low_rank > 0:
            self.pool_w0 = LowRankFastWeight(heads, i_dim, d_dim, cfg.w0_w2_low_rank, cfg.fw_init_gain, True)
            self.pool_w2 = LowRankFastWeight(heads, i_dim, d_dim, cfg.w0_w2_low_rank, cfg.fw_init_gain, True)
        else:
            self.pool_w0 = nn.Parameter(torch.empty(heads, i_dim, d_dim))
            self.pool_w2 = nn.Parameter(torch.empty(heads, i_dim, d_dim))
        self.pool_w1 = nn.Parameter(torch.empty(heads, d_dim, i_dim))
        if cfg.memory_router_share_mode == "share_all" and not self.per_layer_pool:
            self.shared_router_proj_weights = nn.Parameter(torch.empty(1, e, d_dim))
            self.per_layer_router_proj_weights = None
        else:
            self.shared_router_proj_weights = None
            self.per_layer_router_proj_weights = nn.Parameter(torch.empty(cfg.num_hidden_layers, 1, e, d_dim))

    def _init_loss_free_buffers(self) -> None:
        cfg = self.config
        shape = (self.num_experts,) if (cfg.memory_lb_scope == "pool" and not self.per_layer_pool) \
            else (cfg.num_hidden_layers, self.num_experts)
        # the auxiliary-loss-only family has no balancing state in its checkpoints
        # (uttt_llm/flame/custom_models/ttt_moe_no_lb/modeling_recurrent_lact.py registers none)
        keep = getattr(cfg, "model_type", "") != "ttt_moe_no_lb"
        self.register_buffer("memory_loss_free_bias", torch.zeros(shape, dtype=torch.float32), persistent=keep)
        self.register_buffer("memory_loss_free_pending_counts", torch.zeros(shape, dtype=torch.float32),
                             persistent=False)
        self.register_buffer("memory_loss_free_steps", torch.zeros((), dtype=torch.long), persistent=keep)
        self.register_buffer("memory_loss_free_num_updates", torch.zeros((), dtype=torch.long), persistent=keep)
        # device-side flag: 1.0 once any count is pending (keeps the update free of host syncs)
        self._host_steps = 0

    def reset_parameters(self) -> None:
        cfg = self.config
        init_linear_weights(self, cfg.initializer_range)
        for layer in self.layers:
            if layer.memory is not None:
                layer.memory.reset_parameters()
        if not cfg.use_memory_block:
            return
        d_dim, i_dim = cfg.fw_head_dim, cfg.fw_inter_dim
        if cfg.w0_w2_low_rank > 0:
            self.pool_w0.reset_parameters()
            self.pool_w2.reset_parameters()
        else:
            nn.init.normal_(self.pool_w0, std=d_dim ** -0.5)
            nn.init.normal_(self.pool_w2, std=d_dim ** -0.5)
        nn.init.normal_(self.pool_w1, std=i_dim ** -0.5)
        router = self.shared_router_proj_weights if self.shared_router_proj_weights is not None \
            else self.per_layer_router_proj_weights
        nn.init.normal_(router, std=d_dim ** -0.5)

    def _apply(self, fn, *args, **kwargs):
        module = super()._apply(fn, *args, **kwargs)
        for name in ("memory_loss_free_bias", "memory_loss_free_pending_counts"):
            buf = self._buffers.get(name)
            if buf is not None and buf.dtype != torch.float32:
                self._buffers[name] = buf.float()
        return module

    # ------------------------------------------------------------------ helpers
    def _router(self, layer_idx: int) -> torch.Tensor:
        if self.shared_router_proj_weights is not None:
            return self.shared_router_proj_weights[0]
        return self.per_layer_router_proj_weights[layer_idx, 0]

    def _loss_free_enabled(self) -> bool:
        cfg = self.config
        return cfg.memory_lb_mode == "loss_free" and cfg.memory_loss_free_update_rate > 0 and self.num_experts > 1

    def _router_bias(self, layer_idx: int) -> Optional[torch.Tensor]:
        if not self._loss_free_enabled():
            return None
        bias = self.memory_loss_free_bias
        return bias if bias.dim() == 1 else bias[layer_idx]

    def _pool_weights(self):
        cfg = self.config
        w0 = self.pool_w0() if cfg.w0_w2_low_rank > 0 else self.pool_w0
        w2 = self.pool_w2() if cfg.w0_w2_low_rank > 0 else self.pool_w2
        return w0, self.pool_w1, w2

    def compute_dtype(self) -> torch.dtype:
        return self.embeddings.weight.dtype if self.embeddings.weight.dtype != torch.float32 else (
            torch.float32)

    def set_expert_parallel(self, ep) -> None:
        """Shard the experts of the pool over the ranks of ``ep`` (parallel/expert_parallel.py): this rank then
        keeps the state of every sequence of the group for its own experts only."""
        if ep is not None and ep.P > 1:
            if self.per_layer_pool:
                raise NotImplementedError("expert parallelism covers the shared pool (aggregated or chained writes)")

        else:
            ep = None
        self.ep = ep
        for layer in self.layers:
            layer.ep = ep

    def init_states(self, batch: int) -> List[fw.PoolState]:
        """One state for the shared pool, or one per layer for layer-local pools."""
        cfg = self.config
        w0, w1, w2 = self._pool_weights()
        dt = self.compute_dtype()
        e = self.num_experts
        if self.ep is not None:
            mine = self.ep.local_experts()
            return [fw.init_pool_state(w0[mine], w1[mine], w2[mine], batch * self.ep.P, cfg.use_momentum, dt)]
        n_pools = cfg.num_hidden_layers if self.per_layer_pool else 1
        return [fw.init_pool_state(w0[p * e:(p + 1) * e], w1[p * e:(p + 1) * e], w2[p * e:(p + 1) * e], batch,
                                   cfg.use_momentum, dt) for p in range(n_pools)]

    # ------------------------------------------------------------------ loss-free balancing
    @torch.no_grad()
    def _maybe_update_loss_free_bias(self) -> None:
        """bias += u * sign(mean - count) once per update interval; no host sync
        (modeling_recurrent_lact.py:1662-1693)."""
        if not self.training or not self._loss_free_enabled():
            return
        cfg = self.config
        steps = self._host_steps
        counts = self.memory_loss_free_pending_counts
        if steps == 0:
            return
        if steps <= cfg.memory_loss_free_warmup_steps:
            counts.zero_()
            return
        if (steps - cfg.memory_loss_free_warmup_steps) % cfg.memory_loss_free_update_interval != 0:
            return
        bias = self.memory_loss_free_bias
        active = (counts.sum() > 0).to(bias.dtype)
        target = counts.mean() if counts.dim() == 1 else counts.mean(dim=-1, keepdim=True)
        new_bias = bias + cfg.memory_loss_free_update_rate * torch.sign(target - counts)
        new_bias = new_bias - (new_bias.mean() if bias.dim() == 1 else new_bias.mean(dim=-1, keepdim=True))
        if cfg.memory_loss_free_bias_max >= 0:
            new_bias = new_bias.clamp(-cfg.memory_loss_free_bias_max, cfg.memory_loss_free_bias_max)
        bias.copy_(active * new_bias + (1 - active) * bias)
        counts.zero_()
        self.memory_loss_free_num_updates.add_(active.long())

    # ------------------------------------------------------------------ host-side decisions (for graph replay)
    def host_branch_key(self):
        """The decisions the next training forward takes on the host.  A captured CUDA graph of the step replays
        the device work of exactly these decisions; ``None`` means the forward must run eagerly (it reads values
        back for the pool statistics)."""
        cfg = self.config
        if not cfg.use_memory_block:
            return ()
        from . import moe_stats as ms
        if self.num_experts > 1 and self.training and ms.stats_enabled():
            return None
        branch = 0
        if self.training and self._loss_free_enabled():
            steps, warm = self._host_steps, cfg.memory_loss_free_warmup_steps
            if steps == 0:
                branch = 1
            elif steps <= warm:
                branch = 2
            elif (steps - warm) % cfg.memory_loss_free_update_interval != 0:
                branch = 3
            else:
                branch = 4
        return (branch,)

    def host_state(self):
        return {"host_steps": self._host_steps}

    def load_host_state(self, state) -> None:
        self._host_steps = int(state["host_steps"])

    def pop_capture_record(self):
        """What a forward that ran under stream capture left for :meth:`host_step_replayed` (static tensors of the
        captured graph)."""
        record, self._capture_record = getattr(self, "_capture_record", None), None
        return record

    def host_step_replayed(self, record=None) -> None:
        """Bookkeeping of one training forward whose device work was replayed from a graph.  The cross-rank sum of
        the expert counts is not part of the graph (a captured graph holds no collective): it runs here."""
        if self.training and self.config.use_memory_block and self.num_experts > 1 and self._loss_free_enabled():
            if record is not None and record.get("counts") is not None:
                counts = record["counts"].clone()
                if torch.distributed.is_available() and torch.distributed.is_initialized():
                    torch.distributed.all_reduce(counts)
                self.memory_loss_free_pending_counts.add_(counts)
            self._host_steps += 1

    @torch.no_grad()
    def _store_loss_free_counts(self, apply_counts: torch.Tensor, update_counts: torch.Tensor) -> None:
        if not self.training or not self._loss_free_enabled():
            return
        counts = apply_counts.sum(dim=1) + update_counts.sum(dim=1)   # [L, E]
        if self.memory_loss_free_pending_counts.dim() == 1:
            counts = counts.sum(dim=0)
        counts = counts.float()
        self.memory_loss_free_steps.add_(1)
        self._host_steps += 1
        if counts.is_cuda and torch.cuda.is_current_stream_capturing():
            # under graph capture: the sum over ranks and the addition happen after each replay, outside the graph
            self._capture_record = {"counts": counts}
            return
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            torch.distributed.all_reduce(counts)
        self.memory_loss_free_pending_counts.add_(counts)

    # ------------------------------------------------------------------ write
    def _chunk_write(self, states: List[fw.PoolState], feats: List[Tuple[torch.Tensor, ...]], offset: int):
        """Update the bank(s) from this chunk.  Returns (new_states, upd_probs [L,B,E], upd_counts [L,B,E])."""
        cfg = self.config
        mode = cfg.memory_update_backward_mode
        n_layers = len(self.layers)
        dt = states[0].w02.dtype

        if self.per_layer_pool or not cfg.memory_update_aggregate_write:
            # chained writes: every writer applies its own update (to its own pool, or to the shared bank in turn)
            new_states = list(states)
            probs, counts = [], []
            for li, layer in enumerate(self.layers):
                si = li if self.per_layer_pool else 0

                def _one(x_in, k_flat, v_flat, *st, _layer=layer, _li=li):
                    state = fw.PoolState.from_tensors(st)
                    g02, g1, m, p, c = _layer.raw_grad(x_in, k_flat, v_flat, state.w02, state.w1,
                                                       self._router(_li), self._router_bias(_li), offset)
                    if mode in ("first_order_state", "stop_state"):
                        g02, g1 = g02.detach(), g1.detach()
                    if m is not None and (cfg.memory_detach_m_coeff or mode == "stop_state"):
                        m = m.detach()
                    mc = None
                    if m is not None:
                        if self.ep is not None:                  # the owner updates every sequence of the group
                            m = self.ep.gather_sequences(m.reshape(-1))
                        mc = m.view(-1, 1, 1, 1)
                    new = fw.apply_pool_update(g02, g1, state, mc, 1.0, cfg.use_moun, compute_dtype=dt)
                    return (*[t for t in new.tensors() if t is not None], p, c)

                st_in = [t for t in new_states[si].tensors() if t is not None]
                out = self._ckpt(_one, *feats[li], *st_in) if mode != "stop_state" else _one(*feats[li], *st_in)
                n_state = len(st_in)
                vals = list(out[:n_state]) + [None] * (6 - n_state)
                new = fw.PoolState.from_tensors(vals)
                new_states[si] = new.detach() if mode == "stop_state" else new
                probs.append(out[n_state])
                counts.append(out[n_state + 1])
            return new_states, torch.stack(probs), torch.stack(counts)

        state = states[0]
        writers = self.writer_layers
        flat_feats = [t for li in writers for t in feats[li]]
        st_in = [t for t in state.tensors() if t is not None]
        n_state = len(st_in)
        cut = mode == "cross_layer_cut" and self.training and torch.is_grad_enabled()

        def _aggregate(*args):
            f = args[:3 * len(writers)]
            st = list(args[3 * len(writers):]) + [None] * (6 - n_state)
            s = fw.PoolState.from_tensors(st)
            detach_g = mode in ("first_order_state", "stop_state")
            # The aggregate of the first pass over this region (0.9 GB at the 760M shape) is kept for its
            # recomputation, which then records the writers' nodes without redoing their GEMMs and reductions.
            store = self._aggregate_store
            kept = None
            if (store is not None and not detach_g and self.ep is None and torch.is_grad_enabled()
                    and ops.fw_write_accumulate_skips(s.m02, s.w02)):
                kept = store.pop(offset, None)
            else:
                store = None
            if kept is not None:
                a02, a1 = kept
            else:
                a02 = torch.zeros_like(s.m02)
                a1 = torch.zeros_like(s.m1)
            ms, probs, counts = [], [], []
            # the writers' token reductions are added to the aggregate several layers per launch
            stash = None if (detach_g or kept is not None) else ops.write_stash_for(a02)
            for wi, li in enumerate(writers):
                args_l = (f[3 * wi], f[3 * wi + 1], f[3 * wi + 2], s.w02, s.w1, self._router(li),
                          self._router_bias(li), offset)
                if detach_g:
                    g02, g1, m, p, c = self.layers[li].raw_grad(*args_l)
                    a02, a1 = a02 + g02.detach(), a1 + g1.detach()
                else:
                    a02, a1, m, p, c = self.layers[li].raw_grad(
                        *args_l, acc=(a02, a1, stash, wi == len(writers) - 1, kept is not None))
                if m is not None:
                    ms.append(m.detach() if (cfg.memory_detach_m_coeff or mode == "stop_state") else m)
                probs.append(p)
                counts.append(c)
            if store is not None and kept is None:
                store[offset] = (a02.detach(), a1.detach())
            mc = None
            if cfg.memory_aggregate_momentum_mode == "pool_mean" and ms:
                mc = torch.stack(ms, dim=0).mean(dim=0)
                if self.ep is not None:
                    mc = self.ep.gather_sequences(mc.reshape(-1))        # the owner updates every sequence of the group
                mc = mc.view(-1, 1, 1, 1)
            new = fw.apply_pool_update(a02, a1, s, mc, cfg.memory_aggregate_lr_scale, cfg.use_moun, compute_dtype=dt)
            return (*[t for t in new.tensors() if t is not None], torch.stack(probs), torch.stack(counts))

        if cut:
            from .cross_layer_cut import cross_layer_cut_write
            return cross_layer_cut_write(self, states, feats, offset)
        out = _aggregate(*flat_feats, *st_in) if mode == "stop_state" else self._ckpt(_aggregate, *flat_feats, *st_in)
        vals = list(out[:n_state]) + [None] * (6 - n_state)
        new = fw.PoolState.from_tensors(vals)
        if mode == "stop_state":
            new = new.detach()
        e = self.num_experts
        bsz = out[n_state].shape[1]
        probs = torch.zeros(n_layers, bsz, e, device=state.w02.device, dtype=torch.float32)
        counts = torch.zeros_like(probs)
        widx = self._writer_index(probs.device)
        probs = probs.index_copy(0, widx, out[n_state].float())
        counts = counts.index_copy(0, widx, out[n_state + 1].float())
        return [new], probs, counts

    def _writer_index(self, device) -> torch.Tensor:
        cached = getattr(self, "_writer_idx", None)
        if cached is None or cached.device != device:
            cached = torch.tensor(self.writer_layers, device=device)
            self._writer_idx = cached
        return cached

    def _reuse_attention(self, layer_idx: int) -> bool:
        """Whether layer ``layer_idx`` keeps its attention outputs for the recomputation of its regions."""
        return (self.activation_checkpoint and self.training and torch.is_grad_enabled()
                and layer_idx not in self.keep_activation_layers
                and os.environ.get("UTTT_B200_REUSE_ATTENTION", "1") != "0")

    def _ckpt(self, fn, *args):
        if self.activation_checkpoint and torch.is_grad_enabled():
            return checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False)
        return fn(*args)

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: Optional[torch.Tensor] = None, inputs_embeds: Optional[torch.Tensor] = None,
                past_key_values: Any = None, use_cache: bool = False):
        cfg = self.config
        if inputs_embeds is None:
            inputs_embeds = self.embeddings(input_ids)
        if cfg.use_memory_block:
            self._maybe_update_loss_free_bias()
        for layer in self.layers:
            layer.attn.reuse_store = None
        self._aggregate_store = None
        if use_cache and not self.training:
            from .generation import forward_with_cache
            return forward_with_cache(self, inputs_embeds, past_key_values)
        bsz, seq_len, _ = inputs_embeds.shape
        n_layers = len(self.layers)
        chunk = cfg.chunk_size
        e = max(self.num_experts, 1)
        dev = inputs_embeds.device
        states = self.init_states(bsz) if cfg.use_memory_block else []
        hist: List[Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]] = [(None, None)] * n_layers
        keep = self.layers[0].attn.history_len(chunk) if cfg.window_size is not None else None
        apply_probs = torch.zeros(n_layers, bsz, e, device=dev, dtype=torch.float32)
        apply_counts = torch.zeros_like(apply_probs)
        update_probs = torch.zeros_like(apply_probs)
        update_counts = torch.zeros_like(apply_probs)
        cut = (cfg.use_memory_block and cfg.memory_update_backward_mode == "cross_layer_cut" and self.training
               and torch.is_grad_enabled() and not self.per_layer_pool)
        if cut:
            # one aliased copy of the bank per reader layer: reader l's gradient reaches only writer l
            from .cross_layer_cut import alias_streams
            states = alias_streams(states[0], n_layers)
        outputs = []
        sink = (cfg.use_memory_block and not self.per_layer_pool and not cut and self.ep is None and self.training
                and torch.is_grad_enabled())
        if sink:
            ops.reset_grad_sinks()
        # pool statistics every N optimizer steps (models/moe_stats.py); collected in this pass only, not when
        # backward recomputes a region
        from . import moe_stats as ms
        collect = cfg.use_memory_block and self.num_experts > 1 and self.training and ms.stats_enabled()
        routes = (ms.RouteStats(), ms.RouteStats()) if collect else None
        self._aggregate_store = {} if (self._reuse_attention(-1) and cfg.memory_update_backward_mode == "full"
                                       and os.environ.get("UTTT_B200_REUSE_AGGREGATE", "1") != "0") else None
        for li, layer in enumerate(self.layers):
            layer.route_stats = routes
            layer.attn.reuse_store = {} if self._reuse_attention(li) else None
            layer.write_recomputed = cfg.memory_update_backward_mode not in ("stop_state", "cross_layer_cut")
        for start in range(0, seq_len, chunk):
            end = min(start + chunk, seq_len)
            h = inputs_embeds[:, start:end]
            if sink:
                # all readers and writers of this chunk add their bank gradients into one buffer (see ops.grad_sink)
                s0 = states[0]
                states = [fw.PoolState(ops.grad_sink(s0.w02), ops.grad_sink(s0.w1), s0.m02, s0.m1, s0.z02, s0.z1)]
            caches = []
            layer_probs, layer_counts = [], []
            for li, layer in enumerate(self.layers):
                if cfg.use_memory_block:
                    st = states[li] if (self.per_layer_pool or cut) else states[0]
                    w02, w1 = st.w02, st.w1
                    router, bias = self._router(li), self._router_bias(li)
                else:
                    w02 = w1 = router = bias = None
                k_hist, v_hist = hist[li]
                run = layer.__call__ if li in self.keep_activation_layers else (
                    lambda *a, _layer=layer: self._ckpt(_layer, *a))
                with trace_range(f"chunk{start // chunk}.layer{li}.read"):
                    res = run(h, k_hist, v_hist, w02, w1, router, bias, start)
                h, x_in, k_flat, v_flat, k_rot, v_new, p, c = res[:8]
                hist[li] = trim_history(k_hist, v_hist, k_rot, v_new, keep)
                caches.append({"x_attn_in": x_in, "x_memory_in": res[8] if len(res) > 8 else x_in, "xi_out": h,
                               "attn_k": k_flat, "attn_v": v_flat})
                layer_probs.append(p)
                layer_counts.append(c)
            outputs.append(h)
            if cfg.use_memory_block:
                apply_probs = apply_probs + torch.stack(layer_probs)
                apply_counts = apply_counts + torch.stack(layer_counts)
                if end < seq_len:   # apply-then-update; the last chunk never writes
                    with trace_range(f"chunk{start // chunk}.write"):
                        states, up, uc = self._chunk_write(states, self.compose_write_inputs(caches), start)
                    update_probs = update_probs + up
                    update_counts = update_counts + uc
        for layer in self.layers:
            layer.route_stats = None
        hidden = self.norm(torch.cat(outputs, dim=1))
        lb_loss = hidden.new_zeros((), dtype=torch.float32)
        stats = None
        if cfg.use_memory_block and self.num_experts > 1:
            scope = "layer" if self.per_layer_pool else cfg.memory_lb_scope
            apply_lb = fw.lb_loss_for_scope(apply_probs, apply_counts, scope, self.num_experts)
            update_lb = fw.lb_loss_for_scope(update_probs, update_counts, scope, self.num_experts)
            if cfg.memory_lb_mode == "loss":
                lb_loss = (apply_lb + update_lb) * cfg.memory_lb_loss_alpha
            self._store_loss_free_counts(apply_counts, update_counts)
            stats = {"apply_lb": apply_lb.detach(), "update_lb": update_lb.detach(),
                     "apply_counts": apply_counts.detach(), "update_counts": update_counts.detach()}
            if collect:
                stats["moe"] = ms.build_moe_stats(self, apply_lb, update_lb, lb_loss, apply_counts, update_counts,
                                                  routes[0], routes[1])
        return hidden, lb_loss, stats


class UTTTMoEForCausalLM(nn.Module):
    """Causal LM head over :class:`UTTTMoEModel`; ``forward(input_ids, labels)`` returns loss = CE + lb."""

    config_class = None
    model_cls = UTTTMoEModel

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = self.model_cls(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        nn.init.normal_(self.lm_head.weight, std=config.initializer_range)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embeddings.weight

    def forward(self, input_ids=None, labels=None, inputs_embeds=None, past_key_values=None, use_cache=None,
                logits_to_keep: int = 0, return_logits: Optional[bool] = None) -> CausalLMOutput:
        use_cache = bool(use_cache) if use_cache is not None else (self.config.use_cache and not self.training
                                                                   and past_key_values is not None)
        out = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, past_key_values=past_key_values,
                         use_cache=use_cache)
        cache = None
        if len(out) == 4:
            hidden, lb_loss, stats, cache = out
        else:
            hidden, lb_loss, stats = out
        want_logits = return_logits if return_logits is not None else labels is None
        logits = None
        if want_logits:
            hs = hidden[:, -logits_to_keep:] if logits_to_keep else hidden
            logits = self.lm_head(hs)
        loss = ce = None
        if labels is not None:
            # next-token targets: shift inside, last position ignored
            tgt = torch.cat([labels[:, 1:], torch.full_like(labels[:, :1], -100)], dim=1)
            ce = ops.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), self.lm_head.weight,
                                          tgt.reshape(-1), ignore_index=-100)
            loss = ce + lb_loss.to(ce.dtype)
        return CausalLMOutput(loss=loss, logits=logits, ce_loss=None if ce is None else ce.detach(),
                              lb_loss=lb_loss.detach(), hidden_states=hidden, moe_stats=stats,
                              past_key_values=cache)

    # HF-flavoured conveniences -------------------------------------------------------
    @classmethod
    def from_config(cls, config):
        return cls(config)

    def num_parameters(self, exclude_embeddings: bool = False) -> int:
        n = sum(p.numel() for p in self.parameters())
        if exclude_embeddings:
            n -= self.model.embeddings.weight.numel()
        return n


class TTTMoEForCausalLM(UTTTMoEForCausalLM):
    """Layer-local routed pools (config.memory_pool_mode = 'per_layer')."""
