"""VGG-19 perceptual loss and LPIPS-style distance for the view-synthesis model and its evaluation.

Behavioural reference: uttt_nvs/models/perceptual_loss.py:9-213 (feature-space L1 over five VGG-19 stages with
fixed stage weights, ImageNet normalisation, inputs in [0, 1]).

The convolutional trunk is defined here; its weights are read from a file because none can be downloaded at
run time: set ``UTTT_VGG19_WEIGHTS`` (or pass ``weights=``) to a ``torchvision`` VGG-19 ``state_dict`` (keys
``features.N.weight``).  ``UTTT_LPIPS_WEIGHTS`` names the five 1x1 linear heads of LPIPS-VGG (keys ``lin{k}.weight``).
Without weights the constructors raise, unless ``allow_random=True`` (pipeline tests only).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

# VGG-19 feature layout: numbers are conv output channels, "M" is a 2x2 max-pool
_VGG19 = [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512]
# ReLU outputs taken as features: relu1_2, relu2_2, relu3_4, relu4_4, relu5_4 (torchvision ``features`` indices)
_TAPS = (3, 8, 17, 26, 35)
_STAGE_WEIGHTS = (1.0 / 2.6, 1.0 / 4.8, 1.0 / 3.7, 1.0 / 5.6, 10.0 / 1.5)


def _vgg19_features() -> nn.Sequential:
    layers: List[nn.Module] = []
    c_in = 3
    for v in _VGG19:
        if v == "M":
            layers.append(nn.MaxPool2d(2, 2))
        else:
            layers += [nn.Conv2d(c_in, v, 3, padding=1), nn.ReLU(inplace=False)]
            c_in = v
    return nn.Sequential(*layers)


class VGG19Features(nn.Module):
    def __init__(self, weights: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        self.features = _vgg19_features()
        path = weights or os.environ.get("UTTT_VGG19_WEIGHTS", "")
        if path:
            sd = torch.load(path, map_location="cpu", weights_only=True)
            sd = {k[len("features."):]: v for k, v in sd.items() if k.startswith("features.")}
            self.features.load_state_dict(sd, strict=True)
        elif not allow_random:
            raise FileNotFoundError("VGG-19 weights are needed for the perceptual loss: set UTTT_VGG19_WEIGHTS to a "
                                    "torchvision vgg19 state_dict file")
        self.register_buffer("mean", torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("std", torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)
        self.eval()

    def forward(self, x: torch.Tensor) -> List[torch.Tensor]:
        x = (x.float() - self.mean) / self.std
        feats = []
        for i, layer in enumerate(self.features):
            x = layer(x)
            if i in _TAPS:
                feats.append(x)
        return feats

    def train(self, mode: bool = True):          # the trunk never leaves eval mode
        return super().train(False)


class PerceptualLoss(nn.Module):
    """sum_k w_k * mean |phi_k(pred) - phi_k(target)| + pixel L1, inputs [n, 3, H, W] in [0, 1]."""

    def __init__(self, weights: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        self.vgg = VGG19Features(weights, allow_random)

    def forward(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        fp = self.vgg(pred)
        with torch.no_grad():
            ft = self.vgg(target)
        loss = F.l1_loss(pred.float(), target.float())
        for w, a, b in zip(_STAGE_WEIGHTS, fp, ft):
            loss = loss + w * F.l1_loss(a, b)
        return loss


class LPIPSVGG(nn.Module):
    """LPIPS distance: unit-normalised VGG features, squared difference, learned 1x1 heads, spatial mean."""

    _CHANNELS = (64, 128, 256, 512, 512)
    _TAPS16 = (3, 8, 15, 22, 29)                 # LPIPS uses VGG-16 stage ends; VGG-19 taps are used when it is absent

    def __init__(self, vgg_weights: Optional[str] = None, lin_weights: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        self.vgg = VGG19Features(vgg_weights, allow_random)
        self.lins = nn.ModuleList([nn.Conv2d(c, 1, 1, bias=False) for c in self._CHANNELS])
        path = lin_weights or os.environ.get("UTTT_LPIPS_WEIGHTS", "")
        if path:
            sd = torch.load(path, map_location="cpu", weights_only=True)
            for k, lin in enumerate(self.lins):
                lin.weight.data.copy_(sd[f"lin{k}.weight"].view_as(lin.weight))
        elif not allow_random:
            raise FileNotFoundError("LPIPS linear heads are needed: set UTTT_LPIPS_WEIGHTS")
        for p in self.parameters():
            p.requires_grad_(False)
        self.eval()

    @torch.no_grad()
    def forward(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        # LPIPS expects [-1, 1] inputs with its own scaling; the trunk here normalises [0, 1] inputs
        total = 0.0
        for lin, a, b in zip(self.lins, self.vgg(pred), self.vgg(target)):
            a = a / (a.norm(dim=1, keepdim=True) + 1e-10)
            b = b / (b.norm(dim=1, keepdim=True) + 1e-10)
            total = total + lin((a - b) ** 2).mean(dim=(1, 2, 3))
        return total


def build_lpips(device: str = "cpu") -> LPIPSVGG:
    return LPIPSVGG().to(device)
