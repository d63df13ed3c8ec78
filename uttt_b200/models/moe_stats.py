"""Observability of the routed fast-weight pool.

The statistics the reference trainer logs under ``moe/*`` (uttt_llm/flame/custom_models/uttt_moe/
modeling_recurrent_lact.py:178-219, 1926-2017, 3091-3160): balance losses, the state of loss-free balancing
(bias abs-max / std, pending counts, steps, updates), expert usage over the pool and per layer (min / max / std /
coefficient of variation / share of "dead" experts below a quarter of uniform / entropy), and, for reads ("apply")
and writes ("update") separately, the selected combine weights (mean / min / max / median / 95th percentile) and the
router entropy.

They are taken every ``UTTT_MOE_STATS_INTERVAL`` optimizer steps (default 1000; the reference's
``LACT_GLOBAL_MOE_V45_MOE_STATS_INTERVAL`` is honoured too), keyed on the ``FLAME_TRAIN_STEP`` environment variable
that the trainer sets, because the route statistics cost an extra softmax over the router logits.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch


def stats_interval() -> int:
    for name in ("UTTT_MOE_STATS_INTERVAL", "LACT_GLOBAL_MOE_V45_MOE_STATS_INTERVAL",
                 "LACT_GLOBAL_MOE_V45_ROUTE_STATS_INTERVAL"):
        if os.environ.get(name):
            return max(1, int(os.environ[name]))
    return 1000


def stats_enabled() -> bool:
    interval = stats_interval()
    if interval <= 1:
        return True
    step = int(os.environ.get("FLAME_TRAIN_STEP", "0") or "0")
    return step > 0 and step % interval == 0


class RouteStats:
    """Running sums of one kind of routing decision (reads or writes) over the layers and chunks of a forward."""

    def __init__(self):
        self.acc: Optional[Dict[str, torch.Tensor]] = None

    @torch.no_grad()
    def add(self, rows: torch.Tensor, router: torch.Tensor, weights: torch.Tensor) -> None:
        """rows [B, N, D] routed inputs, router [E, D], weights [B*N, k] combine weights of the selected experts."""
        w = weights.detach().float().reshape(-1)
        logits = rows.detach().float().reshape(-1, rows.shape[-1]) @ router.detach().float().t()
        p = torch.softmax(logits, dim=-1)
        entropy = -(p * p.clamp_min(1e-12).log()).sum(-1)
        q = torch.quantile(w, torch.tensor([0.5, 0.95], device=w.device)) if w.numel() else w.new_zeros(2)
        new = {"selected_weight_sum": w.sum(), "selected_weight_count": w.new_tensor(float(w.numel())),
               "selected_weight_min": w.min() if w.numel() else w.new_zeros(()),
               "selected_weight_max": w.max() if w.numel() else w.new_zeros(()),
               "selected_weight_p50_sum": q[0] * w.numel(), "selected_weight_p95_sum": q[1] * w.numel(),
               "router_entropy_sum": entropy.sum(), "router_entropy_count": w.new_tensor(float(entropy.numel()))}
        if self.acc is None:
            self.acc = new
            return
        for k, v in new.items():
            if k.endswith("_min"):
                self.acc[k] = torch.minimum(self.acc[k], v)
            elif k.endswith("_max"):
                self.acc[k] = torch.maximum(self.acc[k], v)
            else:
                self.acc[k] = self.acc[k] + v

    def finalize(self, prefix: str) -> Dict[str, torch.Tensor]:
        if self.acc is None:
            return {}
        a = self.acc
        n = a["selected_weight_count"].clamp_min(1.0)
        return {f"{prefix}_selected_weight_mean": a["selected_weight_sum"] / n,
                f"{prefix}_selected_weight_min": a["selected_weight_min"],
                f"{prefix}_selected_weight_max": a["selected_weight_max"],
                f"{prefix}_selected_weight_p50": a["selected_weight_p50_sum"] / n,
                f"{prefix}_selected_weight_p95": a["selected_weight_p95_sum"] / n,
                f"{prefix}_router_entropy": a["router_entropy_sum"] / a["router_entropy_count"].clamp_min(1.0)}


def expert_usage_stats(counts: torch.Tensor, num_experts: int, prefix: str) -> Dict[str, torch.Tensor]:
    """counts [L, B, E] routed tokens per (layer, sequence, expert) -> pool-level and per-layer usage statistics."""
    per_layer = counts.detach().float().sum(dim=1)                                  # [L, E]
    zero = per_layer.new_zeros(())
    keys = ("freq_min", "freq_max", "freq_std", "freq_cv", "freq_max_over_uniform", "dead_frac_0p25",
            "pool_freq_entropy", "entropy_ratio", "layer_freq_cv_mean", "layer_freq_cv_max",
            "layer_dead_frac_mean_0p25", "layer_dead_frac_max_0p25")
    total = per_layer.sum()
    uniform = 1.0 / float(num_experts)
    dead = 0.25 * uniform
    layer_f = per_layer / per_layer.sum(dim=1, keepdim=True).clamp_min(1e-9)
    pool_f = per_layer.sum(dim=0)
    pool_f = pool_f / pool_f.sum().clamp_min(1e-9)
    std = pool_f.std(unbiased=False)
    ent = -(pool_f.clamp_min(1e-12) * pool_f.clamp_min(1e-12).log()).sum()
    layer_cv = layer_f.std(dim=1, unbiased=False) / layer_f.mean(dim=1).clamp_min(1e-9)
    layer_dead = (layer_f < dead).float().mean(dim=1)
    vals = (pool_f.min(), pool_f.max(), std, std / pool_f.mean().clamp_min(1e-9), pool_f.max() / uniform,
            (pool_f < dead).float().mean(), ent, ent / (math.log(num_experts) if num_experts > 1 else 1.0),
            layer_cv.mean(), layer_cv.max(), layer_dead.mean(), layer_dead.max())
    has = (total > 0).to(per_layer.dtype)                 # all zeros before anything was routed; no host sync
    return {f"{prefix}_{k}": v * has + zero for k, v in zip(keys, vals)}


def build_moe_stats(model, apply_lb, update_lb, lb_loss, apply_counts, update_counts,
                    apply_routes: Optional[RouteStats], update_routes: Optional[RouteStats]) -> Dict[str, torch.Tensor]:
    cfg = model.config
    t = apply_lb.detach()
    e = model.num_experts

    def const(v):
        return t.new_tensor(float(v))
    out = {"apply_lb_loss": apply_lb.detach(), "update_lb_loss": update_lb.detach(), "lb_loss": lb_loss.detach(),
           "num_experts": const(e), "memory_lb_scope_pool": const(cfg.memory_lb_scope == "pool"),
           "memory_lb_mode_loss": const(cfg.memory_lb_mode == "loss"),
           "memory_lb_mode_loss_free": const(cfg.memory_lb_mode == "loss_free"),
           "memory_lb_mode_none": const(cfg.memory_lb_mode == "none"),
           "loss_free_update_rate": const(cfg.memory_loss_free_update_rate),
           "loss_free_bias_abs_max": model.memory_loss_free_bias.detach().abs().max(),
           "loss_free_bias_std": model.memory_loss_free_bias.detach().float().std(unbiased=False),
           "loss_free_pending_count_sum": model.memory_loss_free_pending_counts.detach().sum(),
           "loss_free_steps": model.memory_loss_free_steps.detach().float(),
           "loss_free_num_updates": model.memory_loss_free_num_updates.detach().float()}
    out.update(expert_usage_stats(apply_counts, e, "apply"))
    out.update(expert_usage_stats(update_counts, e, "update"))
    if apply_routes is not None:
        out.update(apply_routes.finalize("apply"))
    if update_routes is not None:
        out.update(update_routes.finalize("update"))
    return out
