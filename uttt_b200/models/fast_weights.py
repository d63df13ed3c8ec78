"""Fast-weight memory: routed SwiGLU expert pools (and the dense special case E = 1, k = 1).

State layout (per local batch of B sequences, E experts, head dim D, inner dim I):

* ``w02`` [B, E, 2I, D]: gate (W0) and up (W2) matrices stacked on the row axis, kept fused
  for the whole sequence so that one grouped GEMM produces both pre-activations;
* ``w1``  [B, E, D, I]: down projection;
* fp32 master copies and fp32 momentum in the same layouts; the compute copies are bf16 on GPU.

Algorithm (uttt_llm/flame/custom_models/uttt_moe/modeling_recurrent_lact.py):
read ``:296-349`` / ``:572-628``, inner gradient ``:389-451`` (loop oracle) and
``:453-518`` (grouped), aggregate write ``:2381-2546``, update rule ``:754-825``.
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref
from .common import RMSNorm


# the gate of the memory read is applied inside the per-head norm kernel (UTTT_B200_GATED_NORM=0: separate multiply)
_GATED_NORM = os.environ.get("UTTT_B200_GATED_NORM", "1") != "0"


@dataclass
class PoolState:
    w02: torch.Tensor
    w1: torch.Tensor
    m02: torch.Tensor          # fp32 master of w02
    m1: torch.Tensor
    z02: Optional[torch.Tensor]  # momentum buffers (None when momentum is off)
    z1: Optional[torch.Tensor]

    def tensors(self):
        return (self.w02, self.w1, self.m02, self.m1, self.z02, self.z1)

    @staticmethod
    def from_tensors(t):
        return PoolState(*t)

    def detach(self) -> "PoolState":
        return PoolState(*[None if t is None else t.detach() for t in self.tensors()])


def init_pool_state(w0: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, batch: int, momentum: bool,
                    compute_dtype: torch.dtype) -> PoolState:
    """w0, w2: [E, I, D]; w1: [E, D, I] (initial fast weights, differentiable) -> per-sequence state."""
    m02 = torch.cat([w0, w2], dim=1).float().unsqueeze(0).repeat(batch, 1, 1, 1)
    m1 = w1.float().unsqueeze(0).repeat(batch, 1, 1, 1)
    z02 = torch.zeros_like(m02) if momentum else None
    z1 = torch.zeros_like(m1) if momentum else None
    return PoolState(m02.to(compute_dtype), m1.to(compute_dtype), m02, m1, z02, z1)


@dataclass
class Routing:
    plan: ops.GroupPlan
    weights: torch.Tensor       # [B*N, k] combine weights (differentiable)
    prob_sum: torch.Tensor      # [B, E] sum of balance probabilities over tokens
    counts: torch.Tensor        # [B, E] tokens routed to each expert
    ep: object = None           # expert-parallel handle (parallel/expert_parallel.py) and its plan, when sharded
    ep_plan: object = None
    idx: Optional[torch.Tensor] = None   # [B, N, k] selected experts


def route_rows(rows: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], cfg,
               bias_in_logits: bool = False, ep=None, reuse=None) -> Routing:
    """rows: [B, N, D]; router: [E, D] (fp32 logits outside autocast; moe_routing.py:7-75).
    With an expert-parallel handle the routing also carries the cross-rank plan."""
    routing = _route_rows_local(rows, router, bias, cfg, bias_in_logits, reuse)
    if ep is not None and ep.P > 1:
        routing.ep = ep
        routing.ep_plan = ep.plan(routing.plan, routing.idx)
    return routing


def _route_rows_local(rows: torch.Tensor, router: torch.Tensor, bias: Optional[torch.Tensor], cfg,
                      bias_in_logits: bool = False, reuse=None) -> Routing:
    """``reuse = (dict, key)``: routing and layout of the first pass over a region are handed to its recomputation
    (see ops.functional._Router)."""
    bsz, n, _ = rows.shape
    e = router.shape[0]
    k = cfg.memory_num_active_experts
    if e == 1:
        idx = torch.zeros(bsz, n, 1, dtype=torch.long, device=rows.device)
        plan = ops.build_group_plan(idx, 1)
        ones = torch.ones(bsz * n, 1, device=rows.device, dtype=torch.float32)
        return Routing(plan, ones, ones.view(bsz, n).sum(1, keepdim=True), plan.sizes.view(bsz, 1).float(), idx=idx)
    idx, weights, psum = ops.route_topk(rows, router, bias, k, cfg.memory_router_alpha, bias_in_logits,
                                        cfg.memory_router_combine_mode == "topk_renorm", cfg.memory_router_type,
                                        cfg.memory_router_scale, cfg.memory_router_norm_eps,
                                        reuse=None if reuse is None else (reuse[0], (reuse[1], "route")))
    plan = ops.build_group_plan(idx, e, None if reuse is None else (reuse[0], (reuse[1], "plan")))
    return Routing(plan, weights, psum, plan.sizes.view(bsz, e).float(), idx=idx)


def pool_read(q_rows: torch.Tensor, state_w02: torch.Tensor, state_w1: torch.Tensor, routing: Routing) -> torch.Tensor:
    """y = sum_{e in top-k} p_e * W1_e (silu(W0_e q) * W2_e q).  q_rows: [B, N, D] -> [B, N, D]."""
    bsz, n, d = q_rows.shape
    if routing.ep is not None:
        # expert-parallel: rows travel to the owners of their experts; the state holds (source, sequence, local expert)
        ep, eplan = routing.ep, routing.ep_plan
        plan = eplan.owner
        g = plan.num_groups
        w02 = state_w02.reshape(g, state_w02.shape[2], d)
        w1 = state_w1.reshape(g, d, state_w1.shape[3])
        if ep.can_fuse_read(q_rows, w02, w1):
            # rows flow to their owners and back tile by tile (parallel/expert_parallel.py::fused_read)
            return ep.fused_read(q_rows.reshape(bsz * n, d).to(w02.dtype), routing.weights, w02, w1,
                                 eplan).view(bsz, n, d)
        xp = ep.dispatch(q_rows.reshape(bsz * n, d).to(w02.dtype), None, eplan)
        hid = ops.gg_swiglu(xp, w02, plan)
        yp = ops.gg_nt(hid, w1, plan)
        return ep.combine(yp, routing.weights, eplan).view(bsz, n, d)
    plan = routing.plan
    g = plan.num_groups
    w02 = state_w02.reshape(g, state_w02.shape[2], d)
    w1 = state_w1.reshape(g, d, state_w1.shape[3])
    xp = ops.permute_rows(q_rows.reshape(bsz * n, d).to(w02.dtype), plan)
    hid = ops.gg_swiglu(xp, w02, plan)
    yp = ops.gg_nt(hid, w1, plan)
    y = ops.unpermute_rows(yp, plan, routing.weights)
    return y.view(bsz, n, d)


def pool_raw_grad(k_rows: torch.Tensor, v_rows: torch.Tensor, lr_rows: torch.Tensor, state_w02: torch.Tensor,
                  state_w1: torch.Tensor, routing: Routing, acc=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inner gradient (ascent direction) of <f_W(k), p*v> per (sequence, expert), lr-weighted per row.

    k_rows, v_rows: [B, N, D]; lr_rows: [B, N, 3] -> (G02 [B, E, 2I, D], G1 [B, E, D, I]) in fp32.
    With ``acc = (A02, A1)`` the gradients are added to those running sums and the sums are returned;
    ``acc = (A02, A1, stash, last)`` defers the additions of several layers into one launch (ops.WriteStash);
    a fifth element ``True`` says that A02 / A1 already hold the complete sums (kept from the first pass over a
    recomputed region): the node is recorded, the arithmetic is skipped.
    """
    bsz, n, d = k_rows.shape
    inter2 = state_w02.shape[2]
    dt = state_w02.dtype
    if routing.ep is not None:
        ep, eplan = routing.ep, routing.ep_plan
        plan = eplan.owner
        kp = ep.dispatch(k_rows.reshape(bsz * n, d).to(dt), None, eplan)
        vp = ep.dispatch(v_rows.reshape(bsz * n, d).to(dt), routing.weights, eplan)
        lr8 = F.pad(lr_rows.reshape(bsz * n, 3).float(), (0, 5))          # 32-byte rows for the transport
        lrp = ep.dispatch(lr8, None, eplan)[:, :3].contiguous()
    else:
        plan = routing.plan
        kp = ops.permute_rows(k_rows.reshape(bsz * n, d).to(dt), plan)
        # v scaled by its combine weight per routed copy while it is scattered
        vp = ops.permute_rows(v_rows.reshape(bsz * n, d).to(dt), plan, routing.weights)
        lrp = _permute_per_choice(lr_rows.reshape(bsz * n, 1, 3).float().expand(-1, plan.topk, -1), plan)
    g = plan.num_groups
    w02 = state_w02.reshape(g, inter2, d)
    w1 = state_w1.reshape(g, d, inter2 // 2)
    if acc is not None:
        stash, last = (acc[2], acc[3]) if len(acc) > 2 else (None, True)
        skip = bool(acc[4]) if len(acc) > 4 else False
        return ops.fw_write_grad_accumulate(kp, vp, lrp, w02, w1, plan, acc[0], acc[1], stash, last, skip)
    g02, g1 = ops.fw_write_grad(kp, vp, lrp, w02, w1, plan)
    return g02.view(*state_w02.shape[:2], inter2, d), g1.view(*state_w02.shape[:2], d, inter2 // 2)


def _permute_per_choice(x: torch.Tensor, plan: ops.GroupPlan) -> torch.Tensor:
    """x: [R, k, C] with a distinct row per routed copy -> [rows_padded, C]."""
    r, k, c = x.shape
    flat = x.reshape(r * k, c)
    out = flat.new_zeros(plan.rows_padded, c)
    return out.index_copy(0, plan.dest.reshape(-1), flat)


def apply_pool_update(a02: torch.Tensor, a1: torch.Tensor, state: PoolState, m_coeff: Optional[torch.Tensor],
                      lr_scale: float, use_muon: bool, ns_coeffs=ref.NS5_COEFFS, renorm: str = "restore",
                      compute_dtype: torch.dtype = torch.bfloat16) -> PoolState:
    """Momentum -> Newton-Schulz per (sequence, expert, matrix) -> master step -> row renorm -> compute copy.

    renorm: "restore" rescales each row back to its previous norm (LM rule); "unit" normalises
    rows to unit length (view-synthesis rule); "none" leaves the master untouched.
    """
    m02, m1 = state.m02, state.m1
    bsz, e, inter2, d = m02.shape
    z02, z1 = state.z02, state.z1
    if z02 is not None and m_coeff is not None:
        a02 = torch.addcmul(a02, z02, m_coeff.to(a02.dtype))
        a1 = torch.addcmul(a1, z1, m_coeff.to(a1.dtype))
        z02, z1 = a02, a1
    if use_muon:
        d02 = ops.newton_schulz(a02.reshape(bsz * e * 2, inter2 // 2, d), ns_coeffs).reshape(bsz, e, inter2, d)
        d1 = ops.newton_schulz(a1.reshape(bsz * e, d, inter2 // 2), ns_coeffs).reshape(bsz, e, d, inter2 // 2)
    else:
        d02, d1 = a02, a1
    n02, w02 = ops.pool_step(m02, d02, lr_scale, renorm, compute_dtype)
    n1, w1 = ops.pool_step(m1, d1, lr_scale, renorm, compute_dtype)
    return PoolState(w02, w1, n02, n1, z02, z1)


class FastWeightMemory(nn.Module):
    """Per-layer parameters of the memory branch (the pool itself is owned by the model).

    Parameter names follow the reference block: ``qk_scale``, ``qk_offset`` [d, 2],
    ``momentum_proj.0.{weight,bias}``, ``ttt_norm.weight``, ``ttt_scale_proj.{weight,bias}``.
    """

    def __init__(self, config, layer_idx: int, momentum_out: int = 1):
        super().__init__()
        self.config = config
        d = config.hidden_size
        self.fw_heads = config.fw_heads
        self.head_dim = config.fw_head_dim
        self.inter_dim = config.fw_inter_dim
        self.qk_rescale = config.memory_qk_rescale
        if self.qk_rescale:
            self.qk_scale = nn.Parameter(torch.ones(d, 2))
            self.qk_offset = nn.Parameter(torch.zeros(d, 2))
        theta = config.rope_theta if config.same_rope else config.ttt_rope_theta
        self.rope_theta = float(theta) if theta else 0.0
        if self.rope_theta > 0:
            self.rope_dim = config.head_dim if config.same_rope else min(self.head_dim, 256)
        else:
            self.rope_dim = 0
        if config.use_momentum:
            self.momentum_proj = nn.Sequential(nn.Linear(d, momentum_out), nn.Sigmoid())
        else:
            self.momentum_proj = None
        self.learnable_ttt_scale = config.learnable_ttt_scale
        self.ttt_norm = RMSNorm(self.head_dim, eps=1e-5)
        if self.learnable_ttt_scale:
            self.ttt_scale_proj = nn.Linear(d, self.fw_heads)
        self.output_proj = nn.Linear(d, d, bias=False) if config.enable_memory_output_proj else None
        self.norm_type = config.memory_qk_norm_type if config.memory_qk_norm else None
        # dedicated q / k / v projections of the memory, only for the sources that use them (ref_base.py:285-304)
        kv_mode = getattr(config, "memory_kv_mode", "reuse_kv")
        own_proj = getattr(config, "memory_kv_proj", "ttt_kv_proj") == "ttt_kv_proj"
        v_only = (own_proj and kv_mode == "reuse_kv" and getattr(config, "memory_v_compose_mode", None) == "ttt-proj"
                  and getattr(config, "memory_k_compose_mode", None) in (None, "reuse")
                  and getattr(config, "memory_k_gap", None) == 0 and getattr(config, "memory_v_gap", None) is not None)
        self.to_q = self.to_k = self.to_v = None
        if own_proj and kv_mode != "reuse_kv":
            self.to_q = nn.Linear(d, d, bias=False)
            self.to_k = nn.Linear(d, d, bias=False)
            self.to_v = nn.Linear(d, d, bias=False)
        elif v_only:
            self.to_v = nn.Linear(d, d, bias=False)

    def reset_parameters(self) -> None:
        if self.qk_rescale:
            nn.init.ones_(self.qk_scale)
            nn.init.zeros_(self.qk_offset)
        if self.learnable_ttt_scale:
            nn.init.normal_(self.ttt_scale_proj.weight, mean=0.0, std=0.1 / (self.config.hidden_size ** 0.5))
            nn.init.zeros_(self.ttt_scale_proj.bias)

    # ---- q / k / v preprocessing ------------------------------------------------------
    def _prep(self, x: torch.Tensor, column: int, offset: int) -> torch.Tensor:
        scale = self.qk_scale[:, column].contiguous() if self.qk_rescale else None
        shift = self.qk_offset[:, column].contiguous() if self.qk_rescale else None
        return ops.fw_qk_prep(x, scale, shift, self.fw_heads, self.rope_dim, self.rope_theta, offset,
                              self.config.memory_qkv_silu, self.norm_type)

    def prep_query(self, q: torch.Tensor, offset: int) -> torch.Tensor:
        return self._prep(q, 0, offset)

    def prep_key(self, k: torch.Tensor, offset: int) -> torch.Tensor:
        return self._prep(k, 1, offset)

    def prep_value(self, v: torch.Tensor) -> torch.Tensor:
        if self.config.memory_qkv_silu:
            v = F.silu(v)
        if self.config.memory_v_norm:
            v = ops.l2_norm(v) if self.config.memory_norm_type == "l2" else ops.rms_norm(v, None, 1e-5)
        return v

    def head_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[b, l, (h hd)] -> [b, (l h), hd]"""
        b, l, _ = x.shape
        return x.reshape(b, l * self.fw_heads, self.head_dim)

    def finish_read(self, y_rows: torch.Tensor, x_in: torch.Tensor) -> torch.Tensor:
        """Per-head RMSNorm of the memory output, times the learned per-head SiLU gate."""
        b, l, _ = x_in.shape
        y = y_rows.reshape(b, l, self.fw_heads, self.head_dim)
        if self.learnable_ttt_scale:
            gate = F.silu(self.ttt_scale_proj(x_in))                  # [b, l, heads]
            if _GATED_NORM:
                y = ops.rms_norm_gated(y, self.ttt_norm.weight, gate.to(y.dtype), self.ttt_norm.eps)
            else:
                y = self.ttt_norm(y) * gate.unsqueeze(-1).to(y.dtype)
        else:
            y = self.ttt_norm(y)
        y = y.reshape(b, l, -1)
        if self.output_proj is not None:
            y = self.output_proj(y)
        return y

    def momentum_coeff(self, x_in: torch.Tensor) -> Optional[torch.Tensor]:
        if self.momentum_proj is None:
            return None
        return self.momentum_proj(x_in).float().mean(dim=1)  # [b, momentum_out]


def lb_loss_for_scope(accum_probs: torch.Tensor, accum_counts: torch.Tensor, scope: str, num_experts: int):
    """Switch-style balance loss from per-(layer, sequence, expert) sums (modeling_recurrent_lact.py:1834-1871)."""
    if scope == "pool":
        p = accum_probs.sum(dim=(0, 1))
        f = accum_counts.sum(dim=(0, 1))
        return ((p / p.sum().clamp_min(1e-9)) * (f / f.sum().clamp_min(1e-9))).sum() * num_experts
    p = accum_probs.sum(dim=1)
    f = accum_counts.sum(dim=1)
    p = p / p.sum(dim=1, keepdim=True).clamp_min(1e-9)
    f = f / f.sum(dim=1, keepdim=True).clamp_min(1e-9)
    return ((p * f).sum(dim=1) * num_experts).sum()
