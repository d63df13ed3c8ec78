"""LVSM-style decoder-only view-synthesis model.

Per scene: camera rays -> Plucker channels (o, d, o x d) + RGB*2-1 -> 12-channel posed images; pose-only
(target) views carry zero RGB; 8x8 patchify in (ph pw c) order -> Linear -> LayerNorm -> block stack
(:mod:`uttt_b200.nvs.blocks`) -> LayerNorm -> Linear -> un-patchify -> sigmoid; loss = MSE on the target
views (+ load-balance term), PSNR reported (uttt_nvs/models/lvsm_moe.py:22-125 loss, :128-163 rays,
:167-294 model).

Two view layouts are supported:
* ``"autoregressive"`` (the reference's): V views become V-1 (posed input i, pose-only target i+1) pairs;
* ``"inputs_then_targets"``: ``num_input_views`` posed views that write the memory, then the remaining
  views decoded from pose only.
"""
from __future__ import annotations

import importlib
import os
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref
from . import blocks as nvs_blocks
from . import stacks as nvs_stacks
from .schedule import inputs_then_targets_config, parallel_ttt_config

# class paths used by the reference YAML files -> classes of this package
_CLASS_ALIASES = {
    "uttt_nvs.models.uttt_moe_block.MemoryModel": nvs_blocks.MemoryModel,
    "uttt_nvs.models.uttt_moe_partitioned.MemoryModel": nvs_blocks.PartitionedMemoryModel,
    "uttt_nvs.models.uttt_dense_block.MemoryModel": nvs_stacks.UTTTDenseModel,
    "uttt_nvs.models.uttt_dense_partitioned.MemoryModel": nvs_stacks.UTTTDensePartitionedModel,
    "uttt_nvs.models.ttt_dense_block.MemoryModel": nvs_stacks.TTTDenseModel,
    "uttt_nvs.models.transformer_block.MemoryModel": nvs_stacks.TransformerModel,
    "uttt_nvs.models.deltanet_block.MemoryModel": nvs_stacks.DeltaNetModel,
    "uttt_nvs.models.gated_deltanet_block.MemoryModel": nvs_stacks.GatedDeltaNetModel,
    # spellings used by earlier configuration files of this package
    "uttt_nvs.models.transformer_block.TransformerModel": nvs_stacks.TransformerModel,
    "uttt_nvs.models.deltanet_block.DeltaNetModel": nvs_stacks.DeltaNetModel,
    "uttt_nvs.models.gated_deltanet_block.GatedDeltaNetModel": nvs_stacks.GatedDeltaNetModel,
}


def get_obj_by_name(path: str):
    """Resolve a dotted class path (uttt_nvs/models/class_name.py:14-67); reference paths map to this package."""
    if path in _CLASS_ALIASES:
        return _CLASS_ALIASES[path]
    module, _, name = path.rpartition(".")
    if module.startswith("uttt_nvs.models"):
        leaf = module.rsplit(".", 1)[-1]
        for key, cls in _CLASS_ALIASES.items():
            if key.rsplit(".", 2)[-2] == leaf:
                return cls
    return getattr(importlib.import_module(module), name)


def resolve_model_class(path: Optional[str] = None):
    """The class that ``model.class_name`` names.  This package has one view-synthesis model, so the reference's
    ``uttt_nvs.models.lvsm_moe.Images2latent3D`` and this module's ``LVSMModel`` both resolve to it; any other name
    is an error rather than a silent substitution."""
    if not path or path in ("uttt_nvs.models.lvsm_moe.Images2latent3D", f"{__name__}.LVSMModel"):
        return LVSMModel
    raise ValueError(f"model.class_name {path!r} is not defined (known: uttt_nvs.models.lvsm_moe.Images2latent3D, "
                     f"{__name__}.LVSMModel)")


class Patchify(nn.Module):
    def __init__(self, patch: int):
        super().__init__()
        self.patch = patch

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        b, v, c, h, w = x.shape
        p = self.patch
        x = x.view(b, v, c, h // p, p, w // p, p).permute(0, 1, 3, 5, 4, 6, 2)
        return x.reshape(b, v * (h // p) * (w // p), p * p * c)


def _cfg_get(cfg, key, default=None):
    if isinstance(cfg, dict):
        return cfg.get(key, default)
    return getattr(cfg, key, default)


class Views(dict):
    """The per-view fields of one side (inputs or targets) of a batch; entries are also attributes."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc


class LVSMModel(nn.Module):
    """``forward(batch)`` with ``batch = {image [b,v,3,H,W], fxfycxcy [b,v,4], c2w [b,v,4,4]}``."""

    def __init__(self, config: Dict[str, Any]):
        super().__init__()
        self.config = config
        m = config["model"]
        size = m["image_size"]
        self.image_size = (size, size) if isinstance(size, int) else tuple(size)
        self.patch_size = m["patch_size"]
        self.dim = m["dim"]
        self.input_dim = 12
        self.view_layout = m.get("view_layout", "autoregressive")
        self.num_input_views = m.get("num_input_views")
        self.image_tokenizer = nn.Sequential(Patchify(self.patch_size),
                                             nn.Linear(self.input_dim * self.patch_size ** 2, self.dim, bias=False))
        self.transformer_input_layernorm = nn.LayerNorm(self.dim, bias=False)
        block_cls = get_obj_by_name(m["block_config"]["type"])
        self.transformer_blocks = block_cls(layers=m["layers"], dim=self.dim, **dict(m["block_config"].get("params", {})))
        self.image_token_decoder = nn.Sequential(nn.LayerNorm(self.dim, bias=False),
                                                 nn.Linear(self.dim, self.patch_size ** 2 * 3, bias=False))
        tr = config.get("training", {})
        self.lpips_weight = float(tr.get("lpips_loss_weight", 0.0) or 0.0)
        self.perceptual_weight = float(tr.get("perceptual_loss_weight", 0.0) or 0.0)
        # the loss networks are plain attributes, not submodules: they never enter the state dict
        # (uttt_nvs/models/lvsm_moe.py:30-58)
        object.__setattr__(self, "perceptual", None)
        object.__setattr__(self, "lpips", None)
        if self.perceptual_weight > 0:
            from .perceptual import PerceptualLoss
            with torch.random.fork_rng(devices=[]):             # its throw-away initialisation must not move the RNG
                object.__setattr__(self, "perceptual", PerceptualLoss())
        if self.lpips_weight > 0:
            from .perceptual import build_lpips
            with torch.random.fork_rng(devices=[]):
                object.__setattr__(self, "lpips", build_lpips())
        self._l2_only = False
        for mod in self.modules():
            if isinstance(mod, nn.Linear):
                nn.init.normal_(mod.weight, std=0.02)

    def l2_warmup(self, set: bool = True) -> None:
        """While set, the loss is the squared error (+ load-balancing term) alone; the trainer sets it from the global
        pass counter (``training.l2_warmup_steps``), so a resumed run does not warm up again
        (uttt_nvs/models/lvsm_moe.py:60-76)."""
        self._l2_only = bool(set)

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        for net in (self.perceptual, self.lpips):                   # follow the model across devices / dtypes
            if net is not None:
                net._apply(fn)
        return out

    # ------------------------------------------------------------------ tokens
    def build_tokens(self, batch):
        """Returns (tokens [b, views*n, p*p*12], schedule, index of the slots to supervise, target images)."""
        image, fxfycxcy, c2w = batch["image"], batch["fxfycxcy"], batch["c2w"]
        b, v, _, h, w = image.shape
        n_tok = (h // self.patch_size) * (w // self.patch_size)
        dev = image.device
        if self.view_layout == "inputs_then_targets":
            n_in = self.num_input_views or (v - 1)
            order = torch.arange(v, device=dev)
            is_target = order >= n_in
            sched = inputs_then_targets_config(n_in, v - n_in, n_tok)
            sup = torch.arange(n_in, v, device=dev)
            targets = image[:, n_in:]
        else:
            # slots 0,2,4,.. = posed view i; slots 1,3,5,.. = pose-only view i+1
            order = torch.stack([torch.arange(v - 1, device=dev), torch.arange(1, v, device=dev)], 1).reshape(-1)
            is_target = torch.arange(2 * (v - 1), device=dev) % 2 == 1
            sched = parallel_ttt_config(n_tok, n_tok, 2 * (v - 1) * n_tok)
            sup = torch.arange(1, 2 * (v - 1), 2, device=dev)
            targets = image[:, 1:]
        with torch.no_grad():
            tokens = ops.plucker_embed(image.index_select(1, order), fxfycxcy.index_select(1, order),
                                       c2w.index_select(1, order), is_target, self.patch_size)
        return tokens.reshape(b, -1, tokens.shape[-1]), sched, sup, targets, n_tok

    def unpatchify(self, y: torch.Tensor, views: int) -> torch.Tensor:
        b = y.shape[0]
        p = self.patch_size
        hh, ww = self.image_size[0] // p, self.image_size[1] // p
        y = y.view(b, views, hh, ww, p, p, 3).permute(0, 1, 6, 2, 4, 3, 5)
        return y.reshape(b, views, 3, hh * p, ww * p)

    def forward(self, batch: Dict[str, torch.Tensor]) -> Dict[str, Any]:
        tokens, sched, sup, targets, n_tok = self.build_tokens(batch)
        dt = self.image_tokenizer[1].weight.dtype
        x = self.image_tokenizer[1](tokens.to(dt))
        x = ops.layer_norm(x, self.transformer_input_layernorm.weight, None, 1e-5)
        x, lb_loss, infos = self.transformer_blocks(x, {"num_img_tokens": n_tok, "ttt_config": sched})
        b = x.shape[0]
        views = x.shape[1] // n_tok
        # only the supervised slots are decoded to pixels
        xs = x.view(b, views, n_tok, self.dim).index_select(1, sup).reshape(b, -1, self.dim)
        y = ops.layer_norm(xs, self.image_token_decoder[0].weight, None, 1e-5)
        logits = self.image_token_decoder[1](y)
        tgt = targets.float()
        # un-patchify + sigmoid + squared-error sums per view in one pass
        rendering, sse = ops.patch_decode(logits, tgt, sup.numel(), self.image_size[0], self.image_size[1],
                                          self.patch_size)
        pixels = 3 * self.image_size[0] * self.image_size[1]
        mse = sse.sum() / (sse.numel() * pixels)
        loss = mse + lb_loss
        perceptual, lpips_loss = rendering.new_zeros(()), rendering.new_zeros(())
        if self.lpips is not None and not self._l2_only:
            lpips_loss = self.lpips(rendering.flatten(0, 1).float(), tgt.flatten(0, 1).clamp(0, 1)).mean()
            loss = loss + self.lpips_weight * lpips_loss
        if self.perceptual is not None and not self._l2_only:
            perceptual = self.perceptual(rendering.flatten(0, 1), tgt.flatten(0, 1))
            loss = loss + self.perceptual_weight * perceptual
        with torch.no_grad():
            per_view = sse.detach() / pixels
            psnr_loc = (-10.0 * torch.log10(per_view.clamp_min(1e-10))).mean(0)
            psnr = psnr_loc.mean()
        metrics = {"loss": loss, "l2_loss": mse.detach(), "lb_loss": lb_loss.detach(), "psnr": psnr,
                   "psnr_loc": psnr_loc, "perceptual_loss": perceptual.detach(),
                   "lpips_loss": lpips_loss.detach()}
        if infos and isinstance(infos[-1], dict):
            metrics.update({k: v for k, v in infos[-1].items()})
        v = batch["image"].shape[1]
        if self.view_layout == "inputs_then_targets":
            n_in = self.num_input_views or (v - 1)
            cut_in, cut_tg = slice(0, n_in), slice(n_in, v)
        else:
            cut_in, cut_tg = slice(0, v - 1), slice(1, v)
        fields = {k: t for k, t in batch.items() if torch.is_tensor(t) and t.dim() >= 2 and t.shape[1] == v}
        return {"input": Views({k: t[:, cut_in] for k, t in fields.items()}),
                "target": Views({k: t[:, cut_tg] for k, t in fields.items()}),
                "loss_metrics": metrics, "rendering": rendering, "op2block2info": infos}

    @torch.no_grad()
    def save_visuals(self, out_dir: str, result: Dict[str, Any], batch: Optional[Dict[str, torch.Tensor]] = None):
        """Writes ``supervision_<first>_<last>.jpg`` (target | rendering per view, scenes stacked), ``input_...jpg``,
        ``uids.txt`` (scene numbers: last column of ``index``) and returns the images plus a per-view PSNR chart
        (uttt_nvs/models/lvsm.py:242-300).  No plotting library is needed: the chart is drawn with Pillow."""
        from PIL import Image, ImageDraw
        os.makedirs(out_dir, exist_ok=True)
        inp, tgt, ren = result["input"], result["target"], result["rendering"]

        def sheet(t):                                     # [b, v, 3, h, w] -> uint8 [(b h), (v w), 3]
            b, v, c, h, w = t.shape
            arr = t.detach().float().cpu().permute(0, 3, 1, 4, 2).reshape(b * h, v * w, c).numpy()
            return (arr * 255.0).clip(0.0, 255.0).astype("uint8")[..., :3]

        pair = torch.cat((tgt["image"].to(ren.dtype), ren), dim=4)              # target beside rendering
        if "index" in tgt:
            uids = [int(tgt["index"][b, 0, -1]) for b in range(tgt["index"].shape[0])]
        else:
            uids = list(range(ren.shape[0]))
        tag = f"{uids[0]:08}_{uids[-1]:08}"
        supervision = Image.fromarray(sheet(pair))
        supervision.save(os.path.join(out_dir, f"supervision_{tag}.jpg"))
        with open(os.path.join(out_dir, "uids.txt"), "w") as fh:
            fh.write("_".join(f"{u:08}" for u in uids))
        inputs = Image.fromarray(sheet(inp["image"]))
        inputs.save(os.path.join(out_dir, f"input_{tag}.jpg"))
        vals = [float(x) for x in result["loss_metrics"]["psnr_loc"].detach().float().cpu().flatten()]
        w, h, pad = 640, 480, 50
        chart = Image.new("RGB", (w, h), "white")
        draw = ImageDraw.Draw(chart)
        lo, hi = min(vals), max(vals)
        span = (hi - lo) or 1.0
        draw.rectangle((pad, pad, w - pad, h - pad), outline="black")
        pts = [(pad + (w - 2 * pad) * (i / max(len(vals) - 1, 1)), h - pad - (h - 2 * pad) * ((v_ - lo) / span))
               for i, v_ in enumerate(vals)]
        if len(pts) > 1:
            draw.line(pts, fill=(31, 119, 180), width=2)
        for x, y in pts:
            draw.ellipse((x - 3, y - 3, x + 3, y + 3), fill=(31, 119, 180))
        draw.text((w // 2 - 40, 15), "Per-view PSNR", fill="black")
        draw.text((5, pad - 5), f"{hi:.2f}", fill="black")
        draw.text((5, h - pad - 5), f"{lo:.2f}", fill="black")
        draw.text((w // 2 - 40, h - 30), f"View (1->{len(vals)})", fill="black")
        return {"supervision": supervision, "input": inputs, "psnr_loc": chart}

    def get_overview(self) -> Dict[str, int]:
        count = lambda mod: sum(p.numel() for p in mod.parameters() if p.requires_grad)
        return {"image_tokenizer": count(self.image_tokenizer), "transformer": count(self.transformer_blocks),
                "image_token_decoder": count(self.image_token_decoder)}


Images2latent3D = LVSMModel
