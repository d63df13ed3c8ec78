"""Small inspection helpers of the view-synthesis trainer (uttt_nvs/models/debug_utils.py: ``sketch_tensor``,
``log_status``) and the router trace callback of the memory blocks."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch


def sketch_tensor(t: torch.Tensor, name: str = "") -> Dict[str, Any]:
    """Shape, dtype and a few robust statistics of a tensor (no host sync beyond the final ``tolist``)."""
    x = t.detach().float().flatten()
    if x.numel() == 0:
        return {"name": name, "shape": list(t.shape), "dtype": str(t.dtype), "numel": 0}
    finite = torch.isfinite(x)
    xf = x[finite] if bool(finite.any()) else x.new_zeros(1)
    stats = torch.stack([xf.mean(), xf.std(unbiased=False), xf.min(), xf.max(), xf.abs().mean(),
                         (~finite).float().sum()]).tolist()
    return {"name": name, "shape": list(t.shape), "dtype": str(t.dtype), "numel": x.numel(), "mean": stats[0],
            "std": stats[1], "min": stats[2], "max": stats[3], "abs_mean": stats[4], "non_finite": int(stats[5])}


def log_status(tensors: Dict[str, torch.Tensor], printer: Callable[[str], None] = print) -> List[Dict[str, Any]]:
    """One line per tensor: ``name shape dtype mean +- std [min, max] non-finite``."""
    rows = [sketch_tensor(t, n) for n, t in tensors.items() if torch.is_tensor(t)]
    for r in rows:
        if r["numel"]:
            printer(f"{r['name']:40s} {str(r['shape']):24s} {r['dtype']:15s} {r['mean']:+.4e} +- {r['std']:.3e} "
                    f"[{r['min']:+.3e}, {r['max']:+.3e}] non-finite {r['non_finite']}")
    return rows


class RouterTrace:
    """Collects per-call routing statistics of the memory blocks: pass an instance as ``router_trace`` in the
    block info dict (or call it from a hook) with (layer, phase, expert counts [B, E], probability sums [B, E])."""

    def __init__(self, max_records: Optional[int] = 4096):
        self.records: List[Dict[str, Any]] = []
        self.max_records = max_records

    def __call__(self, layer: int, phase: str, counts: torch.Tensor, prob_sum: torch.Tensor) -> None:
        if self.max_records is not None and len(self.records) >= self.max_records:
            return
        c = counts.detach().float()
        total = c.sum(dim=-1, keepdim=True).clamp_min(1)
        self.records.append({"layer": int(layer), "phase": phase, "freq_max": float((c / total).max()),
                             "freq_min": float((c / total).min()),
                             "prob_mean": (prob_sum.detach().float() / total).mean(0).tolist()})

    def summary(self) -> Dict[str, float]:
        if not self.records:
            return {}
        return {"calls": len(self.records), "freq_max": max(r["freq_max"] for r in self.records),
                "freq_min": min(r["freq_min"] for r in self.records)}
