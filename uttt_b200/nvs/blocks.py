"""Decoder block stacks for the view-synthesis model.

``MemoryModel``: per view-chunk, every block does full attention inside the view, a routed
fast-weight *read* of a SwiGLU expert pool, and an MLP; after an "update" chunk the pool is written
(uttt_nvs/models/uttt_moe_block.py: block ``:725-815``, read ``:362-423``, raw gradient ``:589-663``,
write rule ``:665-714``, model ``:818-1524``).  Ownership regimes:

* ``pool_mode="shared"`` (uTTT-MoE): one pool for the whole stack; ``aggregate_write`` sums all layers'
  raw gradients from the same snapshot and writes once, otherwise the layers write in turn;
* ``pool_mode="per_block"`` (TTT-MoE): every block owns a pool;
* ``num_experts=1`` gives the dense variants (uTTT-Dense shared, TTT-Dense per block).

Differences from the language model's rule: rows are *unit-normalised* after every write (the master
is left unnormalised), there is no momentum, Newton-Schulz (when enabled) uses fixed coefficients,
routing is a plain softmax over raw logits with top-k on the logits, and the write inputs are
``k = SiLU(W_k x)``, ``v = SiLU(W_v rmsnorm(x))`` with fp32 learning rates.

Parameter names follow the reference state dict (``pool_w0`` ``[1, E, I, D]``, ``blocks.{i}.memory.
input_proj.0.weight`` ...).
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..models import fast_weights as fw
from ..ops import reference as ref
from .schedule import TTTConfig


class _Cfg:
    """Minimal routing config consumed by :func:`uttt_b200.models.fast_weights.route_rows`."""

    def __init__(self, topk: int, alpha: float):
        self.memory_num_active_experts = topk
        self.memory_router_alpha = alpha
        self.memory_router_type = "softmax"
        self.memory_router_combine_mode = "selected_prob"
        self.memory_router_scale = 0.0
        self.memory_router_norm_eps = 1e-6


class SelfAttention(nn.Module):
    """Full (non-causal) attention over the tokens of one view."""

    def __init__(self, dim: int, head_dim: int):
        super().__init__()
        self.dim, self.head_dim = dim, head_dim
        self.to_qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.to_out = nn.Linear(dim, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, l, _ = x.shape
        h = self.dim // self.head_dim
        # three contiguous outputs of the one q|k|v weight (no strided copies, no zero-filled wide gradient)
        q, k, v = (t.view(b, l, h, self.head_dim) for t in ops.split_linear(x, self.to_qkv.weight, 3))
        o = ops.swa_attention(q, k, v, None, causal=False)
        return self.to_out(o.reshape(b, l, self.dim))


class MLP(nn.Module):
    def __init__(self, dim: int, inter_multi: float):
        super().__init__()
        inter = int(dim * inter_multi)
        self.gate = nn.Linear(dim, inter, bias=False)
        self.up = nn.Linear(dim, inter, bias=False)
        self.down = nn.Linear(inter, dim, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y02 = F.linear(x, torch.cat([self.gate.weight, self.up.weight], dim=0))
        return self.down(ops.swiglu(y02.view(-1, y02.shape[-1])).view(*x.shape[:-1], -1))


class FastWeightMemory(nn.Module):
    """Per-block projections of the memory branch (the pool and routers belong to the model)."""

    def __init__(self, dim: int, fw_inter_multi: float, fw_head_dim: Optional[int] = None, base_lr: float = 0.01,
                 use_muon: bool = True, num_experts: int = 2, num_active_experts: int = 1,
                 sigmoid_router: bool = False, router_alpha: float = 1.0, router_from_v: bool = False,
                 l2_norm: bool = False, use_shared_expert: bool = False, **_unused):
        super().__init__()
        if sigmoid_router:
            raise NotImplementedError("sigmoid routing is not supported")
        self.use_shared_expert = bool(use_shared_expert)
        self.dim = dim
        self.head_dim = fw_head_dim or dim
        self.num_heads = dim // self.head_dim
        self.inter_dim = int(self.head_dim * fw_inter_multi)
        self.use_muon, self.l2_norm, self.router_from_v = use_muon, l2_norm, router_from_v
        self.num_experts = num_experts
        self.route_cfg = _Cfg(num_active_experts, router_alpha)
        self.input_proj = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        self.k_input_proj = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        self.to_v = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        self.to_lr = nn.Linear(dim, 3 * self.num_heads, bias=False)
        self.base_lr_inv = base_lr + math.log(-math.expm1(-base_lr))
        self.output_proj = nn.Linear(dim, dim, bias=False)

    def _rows(self, x: torch.Tensor) -> torch.Tensor:
        b, l, _ = x.shape
        rows = x.reshape(b, l * self.num_heads, self.head_dim)
        if self.l2_norm:
            return F.normalize(rows.float(), dim=-1, eps=1e-5).to(x.dtype)
        return ops.rms_norm(rows, None, 1e-5)

    def _proj_rows(self, proj: nn.Sequential, x: torch.Tensor) -> torch.Tensor:
        """Per-head normalised rows of a (Linear, SiLU) projection.  On the GPU in bf16 the SiLU and the per-head norm
        run in the fused preprocessing kernel of the memory branch (its L2 form divides by |y| + 1e-5 where
        ``F.normalize`` divides by max(|y|, 1e-5): 1e-5 relative at most for rows of ordinary size, far inside
        bf16 rounding)."""
        b, l, _ = x.shape
        if x.is_cuda and x.dtype == torch.bfloat16 and self.head_dim % 8 == 0:
            y = ops.fw_qk_prep(ops.linear(x, proj[0].weight), None, None, self.num_heads, 0, 0.0, 0, True,
                               "l2" if self.l2_norm else "rms")
            return y.reshape(b, l * self.num_heads, self.head_dim)
        return self._rows(proj(x))

    @staticmethod
    def shared_expert_ffn(rows: torch.Tensor, se) -> torch.Tensor:
        """The always-on expert of a layer: an un-routed SwiGLU on every row (uttt_moe_block.py:350-360).
        rows [B, T, D]; se = (sw0 [B, 1, I, D], sw1 [B, 1, D, I], sw2 [B, 1, I, D])."""
        sw0, sw1, sw2 = (t.squeeze(1) for t in se)
        hidden = F.silu(torch.bmm(rows, sw0.transpose(1, 2))) * torch.bmm(rows, sw2.transpose(1, 2))
        return torch.bmm(hidden, sw1.transpose(1, 2))

    @staticmethod
    def shared_expert_grad(k: torch.Tensor, v: torch.Tensor, lr: torch.Tensor, se):
        """Raw update of the always-on expert: the gradient of 1/2 |f(k) - v|^2 per matrix, each scaled by its
        learning rate averaged over the rows of a sequence (uttt_moe_block.py:425-462).  k, v [B, T, D]; lr [B, T, 3]
        (lr0, lr1, lr2) -> (dsw0, dsw1, dsw2) shaped like the weights."""
        sw0, sw1, sw2 = (t.squeeze(1) for t in se)
        gate = torch.bmm(k, sw0.transpose(1, 2))
        up = torch.bmm(k, sw2.transpose(1, 2))
        act = F.silu(gate)
        hidden = act * up
        err = torch.bmm(hidden, sw1.transpose(1, 2)) - v
        d1 = torch.bmm(err.transpose(1, 2), hidden)
        dh = torch.bmm(err, sw1)
        sig = torch.sigmoid(gate)
        dgate = dh * up * (sig * (1.0 + gate * (1.0 - sig)))
        d0 = torch.bmm(dgate.transpose(1, 2), k)
        d2 = torch.bmm((dh * act).transpose(1, 2), k)
        mean = lr.mean(dim=1)                                           # [B, 3]
        scale = [mean[:, i].view(-1, 1, 1).to(d0.dtype) for i in range(3)]
        return (d0 * scale[0]).unsqueeze(1), (d1 * scale[1]).unsqueeze(1), (d2 * scale[2]).unsqueeze(1)

    def read(self, x: torch.Tensor, w02: torch.Tensor, w1: torch.Tensor, router: torch.Tensor, se=None):
        b, l, _ = x.shape
        rows = self._proj_rows(self.input_proj, x)
        routing = fw.route_rows(rows, router, None, self.route_cfg)
        y = fw.pool_read(rows, w02, w1, routing)
        if se is not None:
            y = y + self.shared_expert_ffn(rows, se).to(y.dtype)
        y = ops.rms_norm(y, None, 1e-5).reshape(b, l, self.dim)
        return self.output_proj(y.to(x.dtype)), routing.prob_sum, routing.counts

    def raw_grad(self, pre_k, pre_v, w02, w1, router, acc=None, keep_mask: Optional[torch.Tensor] = None, se=None):
        """Routed raw gradient (added to ``acc`` when given) with its balance sums; with ``se`` (the layer's always-on
        expert) the tuple ends with that expert's three raw gradients in fp32."""
        if se is not None and keep_mask is not None:
            raise ValueError("per-token update masking is unsupported when use_shared_expert=True")
        b, l, _ = pre_k.shape
        k_rows = self._proj_rows(self.k_input_proj, pre_k)
        v_rows = self.to_v(pre_v).reshape(b, l * self.num_heads, self.head_dim)
        lr = F.softplus(F.linear(pre_v.float(), self.to_lr.weight.float()) + self.base_lr_inv)
        if keep_mask is not None:
            lr = lr * keep_mask[..., None].to(lr.dtype)
        lr_rows = lr.reshape(b, l * self.num_heads, 3)
        routing = fw.route_rows(v_rows if self.router_from_v else k_rows, router, None, self.route_cfg)
        g02, g1 = fw.pool_raw_grad(k_rows, v_rows, lr_rows, w02, w1, routing, acc=acc)
        if se is not None:
            d0, d1, d2 = self.shared_expert_grad(k_rows, v_rows.to(k_rows.dtype), lr_rows, se)
            return g02, g1, routing.prob_sum, routing.counts, d0.float(), d1.float(), d2.float()
        return g02, g1, routing.prob_sum, routing.counts


class MemoryBlock(nn.Module):
    def __init__(self, dim: int, attn_head_dim: int = 64, inter_multi: float = 2, **kwargs):
        super().__init__()
        self.dim = dim
        self.ln_attn = nn.RMSNorm(dim, eps=1e-5)
        self.self_attention = SelfAttention(dim, attn_head_dim)
        self.ln_memory = nn.RMSNorm(dim, eps=1e-5)
        self.memory = FastWeightMemory(dim, **kwargs)
        self.ln_mlp = nn.RMSNorm(dim, eps=1e-5)
        self.mlp = MLP(dim, inter_multi)

    def forward(self, x, w02, w1, router, *se):
        x = x + self.self_attention(ops.rms_norm(x, self.ln_attn.weight, 1e-5))
        mem_in = ops.rms_norm(x, self.ln_memory.weight, 1e-5)
        y, probs, counts = self.memory.read(mem_in, w02, w1, router, se if se else None)
        x = x + y
        x = x + self.mlp(ops.rms_norm(x, self.ln_mlp.weight, 1e-5))
        return x, mem_in, probs, counts


def _unit_rows_state(w0, w1, w2, batch: int, dtype) -> fw.PoolState:
    """Initial state: masters are the raw parameters, compute copies are their unit-row views."""
    m02 = torch.cat([w0, w2], dim=2).float().repeat(batch, 1, 1, 1)
    m1 = w1.float().repeat(batch, 1, 1, 1)
    return fw.PoolState(F.normalize(m02, dim=3, eps=1e-5).to(dtype), F.normalize(m1, dim=3, eps=1e-5).to(dtype),
                        m02, m1, None, None)


def apply_unit_update(a02, a1, state: fw.PoolState, use_muon: bool, dtype) -> fw.PoolState:
    bsz, e, inter2, d = state.m02.shape
    if use_muon:
        a02 = ops.newton_schulz(a02.reshape(bsz * e * 2, inter2 // 2, d), ref.NS_FIXED_COEFFS).reshape(state.m02.shape)
        a1 = ops.newton_schulz(a1.reshape(bsz * e, d, inter2 // 2), ref.NS_FIXED_COEFFS).reshape(state.m1.shape)
    n02 = state.m02 + a02.float()
    n1 = state.m1 + a1.float()
    return fw.PoolState(F.normalize(n02, dim=3, eps=1e-5).to(dtype), F.normalize(n1, dim=3, eps=1e-5).to(dtype),
                        n02, n1, None, None)


@torch.no_grad()
def routing_statistics(read_counts: torch.Tensor, write_counts: torch.Tensor, shared_pool: bool) -> Dict[str, torch.Tensor]:
    """Balance figures from the per-(layer, scene, expert) selection counts of the reads and the writes
    (uttt_moe_block.py:1468-1506).  Violation rates: per layer and scene, the largest share of an expert times E minus
    one, and the distance of the smallest share times E from one, averaged.  Frequency extrema: shares of the experts
    over reads and writes together, pooled over the layers of a shared pool (per (layer, expert) otherwise)."""
    e = read_counts.shape[-1]

    def violation(counts):
        share = counts.float() / counts.float().sum(dim=-1, keepdim=True)
        return (share.max(dim=-1).values * e - 1.0).mean(), (share.min(dim=-1).values * e - 1.0).abs().mean()

    read_max, read_min = violation(read_counts)
    write_max, write_min = violation(write_counts)
    freq = (read_counts + write_counts).float().sum(dim=1)
    freq = freq.sum(dim=0) if shared_pool else freq.flatten()
    freq = freq / freq.sum().clamp_min(1e-12)
    return {"apply_max_violation_rate": read_max, "apply_min_violation_rate": read_min,
            "update_max_violation_rate": write_max, "update_min_violation_rate": write_min,
            "moe_freq_max": freq.max(), "moe_freq_min": freq.min()}


class MemoryModel(nn.Module):
    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, load_balancing_loss_alpha: float = 0.01,
                 num_experts: int = 2, fw_head_dim: Optional[int] = None, fw_inter_multi: float = 1,
                 pool_mode: str = "shared", router_share_mode: str = "per_layer", use_shared_expert: bool = False,
                 shared_expert_per_layer: bool = False, aggregate_write: bool = False, apply_ckpt_group: int = 1,
                 update_ckpt_sweep: bool = False, offload_master_states: bool = False, **kwargs):
        super().__init__()
        if pool_mode not in ("shared", "per_block"):
            raise ValueError(f"Invalid pool_mode: {pool_mode}")
        if router_share_mode not in ("per_layer", "share_all"):
            raise ValueError(f"Invalid router_share_mode: {router_share_mode}")
        if aggregate_write and pool_mode != "shared":
            raise ValueError("aggregate_write=True is only supported with pool_mode='shared'.")
        if offload_master_states and not aggregate_write:
            raise ValueError("offload_master_states=True requires aggregate_write=True")
        if int(apply_ckpt_group) < 1 or layers % int(apply_ckpt_group) != 0:
            raise ValueError(f"apply_ckpt_group={apply_ckpt_group} must divide the number of layers ({layers})")
        self.v_gap = v_gap
        self.lb_alpha = load_balancing_loss_alpha
        self.pool_mode, self.router_share_mode, self.aggregate_write = pool_mode, router_share_mode, aggregate_write
        self.num_experts = num_experts
        self.apply_ckpt_group, self.update_ckpt_sweep = int(apply_ckpt_group), bool(update_ckpt_sweep)
        self.offload_master_states = bool(offload_master_states)
        self.offload_bytes, self.offload_copies = 0, 0          # cumulative, as the reference's counters
        head_dim = fw_head_dim if fw_head_dim is not None else dim
        inter = int(head_dim * fw_inter_multi)

        def mk(n_out, n_in, fan):
            return nn.Parameter(torch.randn(1, num_experts, n_out, n_in) / math.sqrt(fan))

        if pool_mode == "shared":
            self.pool_w0, self.pool_w1, self.pool_w2 = mk(inter, head_dim, head_dim), mk(head_dim, inter, inter), \
                mk(inter, head_dim, head_dim)
        else:
            self.block_w0_list = nn.ParameterList([mk(inter, head_dim, head_dim) for _ in range(layers)])
            self.block_w1_list = nn.ParameterList([mk(head_dim, inter, inter) for _ in range(layers)])
            self.block_w2_list = nn.ParameterList([mk(inter, head_dim, head_dim) for _ in range(layers)])
        if router_share_mode == "per_layer":
            self.router_proj_weights_list = nn.ParameterList(
                [nn.Parameter(torch.randn(1, num_experts, head_dim) / math.sqrt(head_dim)) for _ in range(layers)])
        else:
            self.shared_router_proj_weights = nn.Parameter(torch.randn(1, num_experts, head_dim) / math.sqrt(head_dim))
        self.use_shared_expert = bool(use_shared_expert)
        # the always-on expert beside the routed pool (uttt_moe_block.py:922-960): one per layer with
        # ``shared_expert_per_layer`` or with per-block pools, otherwise a single one that every layer reads and
        # writes in turn (``shared_expert_w0/1/2``)
        self.shared_expert_is_per_layer = self.use_shared_expert and (bool(shared_expert_per_layer)
                                                                      or pool_mode == "per_block")
        if self.use_shared_expert:
            if int(apply_ckpt_group) > 1:
                raise NotImplementedError("apply_ckpt_group > 1 with use_shared_expert is not implemented "
                                          "(the reference rejects it too)")
            if aggregate_write and not self.shared_expert_is_per_layer:
                raise ValueError("aggregate_write=True requires shared_expert_per_layer=True when "
                                 "use_shared_expert=True.")

            def se_param(n_out, n_in, fan):
                return nn.Parameter(torch.randn(1, 1, n_out, n_in) / math.sqrt(fan))
            if self.shared_expert_is_per_layer:
                self.shared_expert_w0_list = nn.ParameterList([se_param(inter, head_dim, head_dim) for _ in range(layers)])
                self.shared_expert_w1_list = nn.ParameterList([se_param(head_dim, inter, inter) for _ in range(layers)])
                self.shared_expert_w2_list = nn.ParameterList([se_param(inter, head_dim, head_dim) for _ in range(layers)])
            else:
                self.shared_expert_w0 = se_param(inter, head_dim, head_dim)
                self.shared_expert_w1 = se_param(head_dim, inter, inter)
                self.shared_expert_w2 = se_param(inter, head_dim, head_dim)
        self.blocks = nn.ModuleList([
            MemoryBlock(dim=dim, num_experts=num_experts, fw_head_dim=fw_head_dim, fw_inter_multi=fw_inter_multi,
                        use_shared_expert=use_shared_expert, **kwargs) for _ in range(layers)])
        self.v_layer_idxs = [max(min(i + v_gap, layers - 1), 0) for i in range(layers)] if v_gap is not None else None
        self._update_mask_callback = None
        self.activation_checkpoint = True

    def set_update_mask_callback(self, fn) -> None:
        self._update_mask_callback = fn

    def _router(self, i: int) -> torch.Tensor:
        if self.router_share_mode == "share_all":
            return self.shared_router_proj_weights[0]
        return self.router_proj_weights_list[i][0]

    def _ckpt(self, fn, *args):
        if self.activation_checkpoint and torch.is_grad_enabled():
            return checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False)
        return fn(*args)

    def _master_offload(self):
        """`offload_master_states`: the fp32 master copies that autograd keeps per view-chunk for the update's backward
        wait in pinned host memory between forward and backward (uttt_moe_block.py:24-107)."""
        import contextlib
        from ..utils.activation_offload import offload_activations

        @contextlib.contextmanager
        def scope():
            with offload_activations(min_bytes=4 << 20, enabled=self.offload_master_states, fp32_only=True) as off:
                yield off
            self.offload_bytes += off.bytes_offloaded
            self.offload_copies += off.tensors_offloaded
        return scope()

    def init_states(self, batch: int, dtype) -> List[fw.PoolState]:
        if self.pool_mode == "shared":
            return [_unit_rows_state(self.pool_w0, self.pool_w1, self.pool_w2, batch, dtype)]
        return [_unit_rows_state(self.block_w0_list[i], self.block_w1_list[i], self.block_w2_list[i], batch, dtype)
                for i in range(len(self.blocks))]

    def init_shared_experts(self, batch: int, dtype):
        """Per layer (fast, masters) of the always-on expert, or None.  With a single expert for the whole stack every
        entry is the same pair."""
        if not self.use_shared_expert:
            return None
        if not self.shared_expert_is_per_layer:
            masters = tuple(p.float().repeat(batch, 1, 1, 1) for p in
                            (self.shared_expert_w0, self.shared_expert_w1, self.shared_expert_w2))
            return [(_unit_rows(masters, dtype), masters)] * len(self.blocks)
        out = []
        for i in range(len(self.blocks)):
            masters = tuple(p[i].float().repeat(batch, 1, 1, 1) for p in
                            (self.shared_expert_w0_list, self.shared_expert_w1_list, self.shared_expert_w2_list))
            out.append((_unit_rows(masters, dtype), masters))
        return out

    def forward(self, x: torch.Tensor, info: Dict[str, Any]):
        """x: [b, tokens, dim]; info['ttt_config']: list of TTTConfig(start, end, fast_weight, update, apply)."""
        bsz = x.shape[0]
        n = len(self.blocks)
        dt = x.dtype
        shared = self.pool_mode == "shared"
        states = self.init_states(bsz, dt)
        se_states = self.init_shared_experts(bsz, dt)
        e = self.num_experts
        ap = torch.zeros(n, bsz, e, device=x.device)
        ac = torch.zeros_like(ap)
        up = torch.zeros_like(ap)
        uc = torch.zeros_like(ap)
        outputs = []
        source_view = 0
        for cfg in info["ttt_config"]:
            start, end, update = cfg.start, cfg.end, cfg.update
            xi = x[:, start:end]
            mem_ins, outs = [], []
            probs_l, counts_l = [], []
            # `apply_ckpt_group` consecutive blocks share one recompute region: fewer, larger regions (the reference
            # counts 528 -> ceil(24 / K) * 22 regions per step for its large model, uttt_moe_block.py:850-858)
            k_grp = self.apply_ckpt_group
            for g0 in range(0, n, k_grp):
                idx = list(range(g0, g0 + k_grp))

                per = 6 if se_states is not None else 3          # tensors per block: pool, router (+ always-on expert)

                def _group(x_in, *ws, _idx=idx, _per=per):
                    res = []
                    for j, bi in enumerate(_idx):
                        x_in, m_in, p_, c_ = self.blocks[bi](x_in, *ws[_per * j:_per * (j + 1)])
                        res += [x_in, m_in, p_, c_]
                    return tuple(res)
                ws = []
                for bi in idx:
                    st = states[0] if shared else states[bi]
                    ws += [st.w02, st.w1, self._router(bi)]
                    if se_states is not None:
                        ws += list(se_states[bi][0])
                res = self._ckpt(_group, xi, *ws)
                for j in range(k_grp):
                    xi, mem_in, p, c = res[4 * j:4 * j + 4]
                    mem_ins.append(mem_in)
                    outs.append(xi)
                    probs_l.append(p)
                    counts_l.append(c)
            ap = ap + torch.stack(probs_l)
            ac = ac + torch.stack(counts_l)
            outputs.append(xi)
            if update:
                keep = None
                if self._update_mask_callback is not None:
                    keep = self._update_mask_callback(source_view, start, end, x)
                pre_vs = [outs[self.v_layer_idxs[i]] if self.v_layer_idxs is not None else mem_ins[i]
                          for i in range(n)]
                states, p_u, c_u = self._write(states, mem_ins, pre_vs, keep, dt, se_states)
                up = up + p_u
                uc = uc + c_u
                source_view += 1
        out = torch.cat(outputs, dim=1)
        lb = x.new_zeros((), dtype=torch.float32)
        stats: Dict[str, Any] = {}
        if e > 1:
            lb = (fw.lb_loss_for_scope(ap, ac, "layer", e) + fw.lb_loss_for_scope(up, uc, "layer", e)) * self.lb_alpha
            stats = routing_statistics(ac.detach(), uc.detach(), shared)
        return out, lb, [stats]

    def _write(self, states, mem_ins, pre_vs, keep, dt, se_states=None):
        """Updates the pool state(s); with always-on experts, ``se_states`` is updated in place (one entry per
        layer: each layer's expert takes its own raw gradient, whatever the write mode of the pool)."""
        n = len(self.blocks)
        shared = self.pool_mode == "shared"

        def norm_v(t):
            return ops.rms_norm(t, None, 1e-5)

        if se_states is not None:
            return self._write_with_shared_experts(states, mem_ins, pre_vs, keep, dt, se_states, norm_v)

        if shared and self.aggregate_write:
            st = states[0]
            if not self.update_ckpt_sweep:
                # one recompute region per layer's raw gradient; the update itself runs outside them.  The default
                # of the reference; `update_ckpt_sweep` trades 264 regions for 11 at +743 MiB on its large model
                # (uttt_moe_block.py:850-861).
                a02, a1 = torch.zeros_like(st.m02), torch.zeros_like(st.m1)
                ps, cs = [], []
                for i, block in enumerate(self.blocks):
                    def _raw(k_in, v_in, w02, w1, _b=block, _i=i):
                        return _b.memory.raw_grad(k_in, norm_v(v_in), w02, w1, self._router(_i), keep_mask=keep)
                    g02, g1, p, c = self._ckpt(_raw, mem_ins[i], pre_vs[i], st.w02, st.w1)
                    a02, a1 = a02 + g02, a1 + g1
                    ps.append(p)
                    cs.append(c)
                with self._master_offload():
                    new = apply_unit_update(a02, a1, st, self.blocks[0].memory.use_muon, dt)
                return [new], torch.stack(ps), torch.stack(cs)

            def _agg(w02, w1, m02, m1, *feats):
                a02, a1 = torch.zeros_like(m02), torch.zeros_like(m1)
                ps, cs = [], []
                for i, block in enumerate(self.blocks):
                    a02, a1, p, c = block.memory.raw_grad(feats[i], norm_v(feats[n + i]), w02, w1, self._router(i),
                                                          acc=(a02, a1), keep_mask=keep)
                    ps.append(p)
                    cs.append(c)
                new = apply_unit_update(a02, a1, fw.PoolState(w02, w1, m02, m1, None, None),
                                        self.blocks[0].memory.use_muon, dt)
                return new.w02, new.w1, new.m02, new.m1, torch.stack(ps), torch.stack(cs)

            with self._master_offload():
                out = self._ckpt(_agg, st.w02, st.w1, st.m02, st.m1, *mem_ins, *pre_vs)
            return [fw.PoolState(out[0], out[1], out[2], out[3], None, None)], out[4], out[5]

        new_states = list(states)
        ps, cs = [], []
        for i, block in enumerate(self.blocks):
            si = 0 if shared else i

            def _one(w02, w1, m02, m1, k_in, v_in, _b=block, _i=i):
                g02, g1, p, c = _b.memory.raw_grad(k_in, norm_v(v_in), w02, w1, self._router(_i), keep_mask=keep)
                new = apply_unit_update(g02, g1, fw.PoolState(w02, w1, m02, m1, None, None), _b.memory.use_muon, dt)
                return new.w02, new.w1, new.m02, new.m1, p, c

            s = new_states[si]
            out = self._ckpt(_one, s.w02, s.w1, s.m02, s.m1, mem_ins[i], pre_vs[i])
            new_states[si] = fw.PoolState(out[0], out[1], out[2], out[3], None, None)
            ps.append(out[4])
            cs.append(out[5])
        return new_states, torch.stack(ps), torch.stack(cs)


def _unit_rows(masters, dtype):
    return tuple(F.normalize(m, dim=3, eps=1e-5).to(dtype) for m in masters)


def apply_shared_expert_update(raw, masters, use_muon: bool, dtype):
    """masters += (Newton-Schulz of) raw, then unit rows (uttt_moe_block.py:690-714).  -> (fast, masters)"""
    if use_muon:
        raw = tuple(ops.newton_schulz(g.flatten(0, 1), ref.NS_FIXED_COEFFS).reshape(g.shape) for g in raw)
    new = tuple(m + g.float() for m, g in zip(masters, raw))
    return _unit_rows(new, dtype), new


def _write_with_shared_experts(self, states, mem_ins, pre_vs, keep, dt, se_states, norm_v):
    """The write of :class:`MemoryModel` when every layer has an always-on expert: one recompute region per layer
    returns the routed raw gradient and the expert's; the pool is updated once from the aggregate
    (``aggregate_write``) or layer by layer, every expert from its own gradient (uttt_moe_block.py:1128-1183, 1340-1420)."""
    n = len(self.blocks)
    shared = self.pool_mode == "shared"
    use_muon = self.blocks[0].memory.use_muon
    ps, cs = [], []
    new_states = list(states)
    a02 = a1 = None
    for i, block in enumerate(self.blocks):
        st = new_states[0 if shared else i]

        def _raw(k_in, v_in, w02, w1, s0, s1, s2, _b=block, _i=i):
            return _b.memory.raw_grad(k_in, norm_v(v_in), w02, w1, self._router(_i), keep_mask=keep, se=(s0, s1, s2))
        g02, g1, p, c, d0, d1, d2 = self._ckpt(_raw, mem_ins[i], pre_vs[i], st.w02, st.w1, *se_states[i][0])
        ps.append(p)
        cs.append(c)
        se_states[i] = apply_shared_expert_update((d0, d1, d2), se_states[i][1], use_muon, dt)
        if not self.shared_expert_is_per_layer:
            se_states[:] = [se_states[i]] * n                    # one expert for the stack: the next layer sees this write
        if shared and self.aggregate_write:
            a02, a1 = (g02, g1) if a02 is None else (a02 + g02, a1 + g1)
        else:
            new_states[0 if shared else i] = apply_unit_update(g02, g1, st, block.memory.use_muon, dt)
    if shared and self.aggregate_write:
        with self._master_offload():
            new_states = [apply_unit_update(a02, a1, states[0], use_muon, dt)]
    return new_states, torch.stack(ps), torch.stack(cs)


MemoryModel._write_with_shared_experts = _write_with_shared_experts


class PartitionedMemoryModel(nn.Module):
    """Depth-contiguous groups of blocks, each group with its own shared pool; ``num_experts`` is the total expert
    budget, split evenly over the groups (uttt_nvs/models/uttt_moe_partitioned.py:10-462).

    Parameters and blocks are registered in the reference's flat layout: ``pool_w{0,1,2}_list[p]``, ``blocks[i]``,
    ``pool_router_proj_weights_list[p]`` (``router_share_mode="share_pool"``, one router per group) or
    ``shared_router_proj_weights`` (``"share_all"``, one router for every group), ``shared_expert_w{0,1,2}_list[i]``.
    Each group is run by a :class:`MemoryModel` over its slice of the blocks and its pool; these runners hold the same
    parameter and module objects and are not registered as children.  A group's writes depend on its own blocks only,
    so running group after group over the whole schedule gives what the layer-interleaved walk gives; this needs
    ``v_gap`` to stay inside a group, so ``v_gap`` with more than one group is refused."""

    def __init__(self, layers: int, dim: int, num_partitions: Optional[int] = None, num_experts: int = 4,
                 num_shared_pools: Optional[int] = None, pool_mode: str = "shared",
                 router_share_mode: str = "share_pool", v_gap: Optional[int] = None, **kwargs):
        super().__init__()
        # `num_shared_pools` is the reference's name of the option
        pools = int(num_shared_pools if num_shared_pools is not None else (num_partitions or 1))
        if pools <= 0:
            raise ValueError("num_shared_pools must be positive.")
        if pool_mode != "shared":
            raise ValueError("the partitioned stack only supports pool_mode='shared'.")
        if layers % pools or num_experts % pools:
            raise ValueError("layers and num_experts must be divisible by the number of pools")
        if router_share_mode not in ("share_pool", "share_all"):
            raise ValueError("router_share_mode must be either 'share_pool' or 'share_all'.")
        if v_gap is not None and pools > 1:
            raise NotImplementedError("v_gap across partitions is not built: the groups run one after the other")
        self.num_shared_pools, self.router_share_mode = pools, router_share_mode
        self.pool_size, self.experts_per_pool = layers // pools, num_experts // pools
        runners = [MemoryModel(self.pool_size, dim, num_experts=self.experts_per_pool, pool_mode="shared",
                               router_share_mode="share_all", v_gap=v_gap, **kwargs) for _ in range(pools)]
        self.pool_w0_list = nn.ParameterList([r.pool_w0 for r in runners])
        self.pool_w1_list = nn.ParameterList([r.pool_w1 for r in runners])
        self.pool_w2_list = nn.ParameterList([r.pool_w2 for r in runners])
        if router_share_mode == "share_pool":
            self.pool_router_proj_weights_list = nn.ParameterList([r.shared_router_proj_weights for r in runners])
        else:
            self.shared_router_proj_weights = runners[0].shared_router_proj_weights
            for r in runners[1:]:
                r.shared_router_proj_weights = self.shared_router_proj_weights
        if runners[0].use_shared_expert and not runners[0].shared_expert_is_per_layer:
            raise NotImplementedError("one always-on expert for all pools is not built for the partitioned stack (the "
                                      "groups run one after the other); use shared_expert_per_layer=True")
        if runners[0].use_shared_expert:
            for name in ("shared_expert_w0_list", "shared_expert_w1_list", "shared_expert_w2_list"):
                setattr(self, name, nn.ParameterList([p for r in runners for p in getattr(r, name)]))
        self.blocks = nn.ModuleList([b for r in runners for b in r.blocks])
        object.__setattr__(self, "parts", runners)                   # same objects as above; not registered twice
        self.activation_checkpoint = True

    def set_update_mask_callback(self, fn) -> None:
        for part in self.parts:
            part.set_update_mask_callback(fn)

    def _bind(self) -> None:
        """Points the runners at the registered parameters again (a conversion such as ``to_empty`` replaces the
        parameter objects of this module, which the unregistered runners would not see)."""
        n = self.pool_size
        for p, r in enumerate(self.parts):
            if r.pool_w0 is self.pool_w0_list[p]:
                continue
            r.pool_w0, r.pool_w1, r.pool_w2 = self.pool_w0_list[p], self.pool_w1_list[p], self.pool_w2_list[p]
            r.shared_router_proj_weights = self.pool_router_proj_weights_list[p] \
                if self.router_share_mode == "share_pool" else self.shared_router_proj_weights
            if r.use_shared_expert:
                for name in ("shared_expert_w0_list", "shared_expert_w1_list", "shared_expert_w2_list"):
                    setattr(r, name, nn.ParameterList(list(getattr(self, name))[p * n:(p + 1) * n]))

    def forward(self, x, info):
        self._bind()
        lb_total = x.new_zeros((), dtype=torch.float32)
        infos: List[Any] = []
        # every group sees the whole schedule: group g's output sequence feeds group g+1
        for part in self.parts:
            part.activation_checkpoint = self.activation_checkpoint
            x, lb, inf = part(x, info)
            lb_total = lb_total + lb
            infos = inf
        return x, lb_total, infos
