"""Learning-rate schedules: linear warmup followed by linear / cosine / constant decay to
``lr_min * lr`` (flags ``lr_scheduler.{warmup_steps,decay_ratio,decay_type,lr_min}``,
uttt_llm/flame/config_manager.py:237-290)."""
from __future__ import annotations

import math
from typing import Dict


class WarmupDecayLR:
    def __init__(self, base_lr: float, total_steps: int, warmup_steps: int = 0, decay_type: str = "cosine",
                 lr_min: float = 0.0, decay_ratio: float | None = None):
        if decay_type not in {"linear", "cosine", "sqrt", "constant"}:
            raise ValueError(f"unknown decay_type {decay_type!r}")
        self.base_lr, self.total_steps, self.warmup_steps = base_lr, max(total_steps, 1), warmup_steps
        self.decay_type, self.lr_min = decay_type, lr_min
        decay_steps = self.total_steps - warmup_steps if decay_ratio is None else int(self.total_steps * decay_ratio)
        self.stable_end = self.total_steps - max(decay_steps, 0)
        self.last_step = 0

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            return float(step + 1) / float(self.warmup_steps + 1)
        if self.decay_type == "constant" or step < self.stable_end:
            return 1.0
        span = max(self.total_steps - self.stable_end, 1)
        progress = min(max((step - self.stable_end) / span, 0.0), 1.0)
        if self.decay_type == "linear":
            f = 1.0 - progress
        elif self.decay_type == "sqrt":
            f = 1.0 - math.sqrt(progress)
        else:
            f = 0.5 * (1.0 + math.cos(math.pi * progress))
        return self.lr_min + (1.0 - self.lr_min) * f

    def lr(self) -> float:
        return self.base_lr * self.factor(self.last_step)

    def step(self) -> float:
        self.last_step += 1
        return self.lr()

    def fast_forward(self, step: int) -> None:
        self.last_step = step

    def state_dict(self) -> Dict[str, float]:
        return {"last_step": self.last_step}

    def load_state_dict(self, sd: Dict[str, float]) -> None:
        self.last_step = int(sd["last_step"])
