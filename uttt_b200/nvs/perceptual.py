"""VGG perceptual loss and LPIPS-VGG distance for the view-synthesis model and its evaluation.

* :class:`PerceptualLoss` is the loss of uttt_nvs/models/perceptual_loss.py:9-213: images in [0, 1] are scaled to
  0..255 and the channel means (123.68, 116.779, 103.939) subtracted; a VGG-19 trunk **with average pooling** gives
  the features after ``relu1_2, relu2_2, relu3_2, relu4_2, relu5_2``; the loss is
  ``(|dx| + |d f1| / 2.6 + |d f2| / 4.8 + |d f3| / 3.7 + |d f4| / 5.6 + 10 |d f5| / 1.5) / 255`` with ``|.|`` the mean
  absolute difference.  Weights: the MatConvNet file ``imagenet-vgg-verydeep-19.mat`` that the reference loads
  (``VGG19_MAT_PATH``, read with scipy), or a ``torchvision`` VGG-19 ``state_dict`` (``UTTT_VGG19_WEIGHTS``; other
  trained weights, so other loss values).
* :class:`LPIPSVGG` is LPIPS with the VGG-16 trunk (what ``lpips.LPIPS(net="vgg")`` computes with ``normalize=True``):
  inputs in [0, 1] mapped to [-1, 1], the fixed input scaling layer, features after ``relu1_2, relu2_2, relu3_3,
  relu4_3, relu5_3`` scaled to unit length over channels, squared differences through the learned 1x1 heads, spatial
  means summed over the five stages.  Weights: a ``torchvision`` VGG-16 ``state_dict`` (``UTTT_VGG16_WEIGHTS``) and
  the heads (``UTTT_LPIPS_WEIGHTS``: the ``lpips`` package's ``vgg.pth`` with keys ``lin{k}.model.1.weight``, or
  ``lin{k}.weight``).

Nothing can be downloaded at run time, so every weight comes from a file; without one the constructors raise, unless
``allow_random=True`` (pipeline tests only).  Both modules are differentiable with respect to the prediction.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

# conv output channels per layer, "P" = 2x2 pooling; indices below count conv / relu / pool modules as torchvision does
_VGG19 = [64, 64, "P", 128, 128, "P", 256, 256, 256, 256, "P", 512, 512, 512, 512, "P", 512, 512, 512, 512]
_VGG16 = [64, 64, "P", 128, 128, "P", 256, 256, 256, "P", 512, 512, 512, "P", 512, 512, 512]
_TAPS19_SECOND_RELU = (3, 8, 13, 22, 31)          # relu1_2, relu2_2, relu3_2, relu4_2, relu5_2
_TAPS16_STAGE_ENDS = (3, 8, 15, 22, 29)           # relu1_2, relu2_2, relu3_3, relu4_3, relu5_3
_STAGE_WEIGHTS = (1.0 / 2.6, 1.0 / 4.8, 1.0 / 3.7, 1.0 / 5.6, 10.0 / 1.5)
_MATCONVNET_CONV_LAYERS = (0, 2, 5, 7, 10, 12, 14, 16, 19, 21, 23, 25, 28, 30, 32, 34)


def _trunk(layout: Sequence, pool: str) -> nn.Sequential:
    layers: List[nn.Module] = []
    c_in = 3
    for v in layout:
        if v == "P":
            layers.append(nn.AvgPool2d(2, 2) if pool == "avg" else nn.MaxPool2d(2, 2))
        else:
            layers += [nn.Conv2d(c_in, v, 3, padding=1), nn.ReLU(inplace=False)]
            c_in = v
    return nn.Sequential(*layers)


def load_matconvnet_vgg19(features: nn.Sequential, path: str) -> None:
    """Convolution weights of ``imagenet-vgg-verydeep-19.mat``: ``layers[0][i]`` is a 1x1 struct whose third field
    (``weights``) is a 1x2 cell of the filter bank ``[h, w, in, out]`` and the bias."""
    import scipy.io
    raw = scipy.io.loadmat(path)["layers"][0]
    convs = [m for m in features if isinstance(m, nn.Conv2d)]
    for conv, idx in zip(convs, _MATCONVNET_CONV_LAYERS):
        record = raw[idx][0][0]
        cell = record["weights"] if record.dtype.names and "weights" in record.dtype.names else record[2]
        w, b = cell[0][0], cell[0][1]
        conv.weight.data.copy_(torch.from_numpy(w).permute(3, 2, 0, 1))
        conv.bias.data.copy_(torch.from_numpy(b).reshape(-1))


def _load_torchvision(features: nn.Sequential, path: str) -> None:
    sd = torch.load(path, map_location="cpu", weights_only=True)
    sd = {k[len("features."):]: v for k, v in sd.items() if k.startswith("features.")}
    features.load_state_dict(sd, strict=True)


class _FrozenTrunk(nn.Module):
    def __init__(self, layout, pool: str, taps: Sequence[int]):
        super().__init__()
        self.features = _trunk(layout, pool)
        self.taps = tuple(taps)

    def freeze(self):
        for p in self.parameters():
            p.requires_grad_(False)
        self.eval()

    def stages(self, x: torch.Tensor) -> List[torch.Tensor]:
        feats = []
        for i, layer in enumerate(self.features):
            x = layer(x)
            if i in self.taps:
                feats.append(x)
            if i == self.taps[-1]:
                break
        return feats

    def train(self, mode: bool = True):          # the trunk never leaves eval mode
        return super().train(False)


class VGG19Features(_FrozenTrunk):
    """The perceptual loss's trunk: average pooling, inputs in 0..255 minus the channel means."""

    def __init__(self, weights: Optional[str] = None, allow_random: bool = False):
        super().__init__(_VGG19, "avg", _TAPS19_SECOND_RELU)
        mat = weights if (weights or "").endswith(".mat") else os.environ.get("VGG19_MAT_PATH", "")
        tv = weights if weights and not weights.endswith(".mat") else os.environ.get("UTTT_VGG19_WEIGHTS", "")
        if mat:
            if not os.path.isfile(mat):
                raise FileNotFoundError(f"VGG-19 weights not found at {mat}")
            load_matconvnet_vgg19(self.features, mat)
        elif tv:
            _load_torchvision(self.features, tv)
        elif not allow_random:
            raise FileNotFoundError(
                "VGG-19 weights are needed for the perceptual loss (training.perceptual_loss_weight > 0): set "
                "VGG19_MAT_PATH to imagenet-vgg-verydeep-19.mat (the MatConvNet file the reference uses), or "
                "UTTT_VGG19_WEIGHTS to a torchvision vgg19 state_dict file")
        self.register_buffer("mean", torch.tensor([123.6800, 116.7790, 103.9390]).view(1, 3, 1, 1), persistent=False)
        self.freeze()

    def scale(self, x: torch.Tensor) -> torch.Tensor:
        return x.float() * 255.0 - self.mean

    def forward(self, x: torch.Tensor) -> List[torch.Tensor]:
        return self.stages(self.scale(x))


class PerceptualLoss(nn.Module):
    """Pixel L1 plus weighted feature L1 over five VGG-19 stages, inputs [n, 3, H, W] in [0, 1]."""

    def __init__(self, weights: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        self.vgg = VGG19Features(weights, allow_random)

    def forward(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        p, t = self.vgg.scale(pred), self.vgg.scale(target)
        fp = self.vgg.stages(p)
        with torch.no_grad():
            ft = self.vgg.stages(t)
        loss = (t - p).abs().mean()
        for w, a, b in zip(_STAGE_WEIGHTS, fp, ft):
            loss = loss + w * (b - a).abs().mean()
        return loss / 255.0


class LPIPSVGG(nn.Module):
    """LPIPS-VGG distance per image, inputs [n, 3, H, W] in [0, 1]."""

    _CHANNELS = (64, 128, 256, 512, 512)

    def __init__(self, vgg_weights: Optional[str] = None, lin_weights: Optional[str] = None, allow_random: bool = False):
        super().__init__()
        self.vgg = _FrozenTrunk(_VGG16, "max", _TAPS16_STAGE_ENDS)
        self.lins = nn.ModuleList([nn.Conv2d(c, 1, 1, bias=False) for c in self._CHANNELS])
        trunk = vgg_weights or os.environ.get("UTTT_VGG16_WEIGHTS", "")
        heads = lin_weights or os.environ.get("UTTT_LPIPS_WEIGHTS", "")
        if trunk:
            _load_torchvision(self.vgg.features, trunk)
        elif not allow_random:
            raise FileNotFoundError("LPIPS needs the VGG-16 trunk: set UTTT_VGG16_WEIGHTS to a torchvision vgg16 "
                                    "state_dict file")
        if heads:
            sd = torch.load(heads, map_location="cpu", weights_only=True)
            for k, lin in enumerate(self.lins):
                w = sd[f"lin{k}.model.1.weight"] if f"lin{k}.model.1.weight" in sd else sd[f"lin{k}.weight"]
                lin.weight.data.copy_(w.view_as(lin.weight))
        elif not allow_random:
            raise FileNotFoundError("LPIPS linear heads are needed: set UTTT_LPIPS_WEIGHTS (the lpips package's vgg.pth)")
        self.register_buffer("shift", torch.tensor([-0.030, -0.088, -0.188]).view(1, 3, 1, 1), persistent=False)
        self.register_buffer("scale", torch.tensor([0.458, 0.448, 0.450]).view(1, 3, 1, 1), persistent=False)
        for p in self.parameters():
            p.requires_grad_(False)
        self.eval()

    def _features(self, x: torch.Tensor) -> List[torch.Tensor]:
        x = (2.0 * x.float() - 1.0 - self.shift) / self.scale
        return [f / (f.pow(2).sum(dim=1, keepdim=True).sqrt() + 1e-10) for f in self.vgg.stages(x)]

    def forward(self, pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        total = 0.0
        for lin, a, b in zip(self.lins, self._features(pred), self._features(target)):
            total = total + lin((a - b) ** 2).mean(dim=(1, 2, 3))
        return total

    def train(self, mode: bool = True):
        return super().train(False)


def build_lpips(device: str = "cpu") -> LPIPSVGG:
    return LPIPSVGG().to(device)
