"""Image metrics and scene-bootstrap statistics for the view-synthesis evaluation
(uttt_nvs/eval/metrics.py:9-86, statistics.py)."""
from __future__ import annotations

from typing import Dict, Sequence

import numpy as np
import torch
import torch.nn.functional as F


def psnr(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """[..., 3, H, W] in [0, 1] -> PSNR per leading index."""
    mse = ((pred.float() - target.float()) ** 2).mean(dim=(-3, -2, -1))
    return -10.0 * torch.log10(mse.clamp_min(1e-10))


def ssim(pred: torch.Tensor, target: torch.Tensor, window: int = 11, sigma: float = 1.5) -> torch.Tensor:
    """Gaussian-window SSIM per image for [n, 3, H, W] in [0, 1]."""
    ax = torch.arange(window, dtype=torch.float32, device=pred.device) - window // 2
    g = torch.exp(-(ax ** 2) / (2 * sigma ** 2))
    g = g / g.sum()
    k = (g[:, None] * g[None, :]).expand(3, 1, window, window).contiguous()
    p, t = pred.float(), target.float()
    mu_p, mu_t = F.conv2d(p, k, groups=3), F.conv2d(t, k, groups=3)
    s_pp = F.conv2d(p * p, k, groups=3) - mu_p ** 2
    s_tt = F.conv2d(t * t, k, groups=3) - mu_t ** 2
    s_pt = F.conv2d(p * t, k, groups=3) - mu_p * mu_t
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    m = ((2 * mu_p * mu_t + c1) * (2 * s_pt + c2)) / ((mu_p ** 2 + mu_t ** 2 + c1) * (s_pp + s_tt + c2))
    return m.mean(dim=(1, 2, 3))


def bootstrap_ci(per_scene: Sequence[float], resamples: int = 10000, seed: int = 9595,
                 level: float = 0.95) -> Dict[str, float]:
    """Mean with a percentile bootstrap interval over scenes."""
    x = np.asarray(per_scene, dtype=np.float64)
    rng = np.random.default_rng(seed)
    idx = rng.integers(0, len(x), size=(resamples, len(x)))
    means = x[idx].mean(axis=1)
    lo, hi = np.quantile(means, [(1 - level) / 2, 1 - (1 - level) / 2])
    return {"mean": float(x.mean()), "ci_low": float(lo), "ci_high": float(hi), "n": int(len(x))}
