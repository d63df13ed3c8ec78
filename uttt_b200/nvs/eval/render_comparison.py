"""Side-by-side comparison sheets of several registry entries (uttt_nvs/eval/render_comparison.py).

    python -m uttt_b200.nvs.eval.render_comparison --registry R --dataset gso --experiment A --experiment B \
        [--scene-id S ...] [--scene-count 8] [--view-indices 1,12,23] [--seed 9595] [--device cuda:0] \
        [--amp-dtype bf16] --output-root DIR [--allow-missing-checkpoint]

Per chosen scene a folder ``<output-root>/<dataset>/<scene>/`` with ``input_view_00.png``,
``ground_truth_view_<k>.png``, ``<model>_view_<k>.png`` and ``comparison.png``: one row per chosen view k, columns =
the latest conditioning view (k - 1), the ground truth of view k, then one column per model with its PSNR / SSIM / LPIPS
for that view underneath.  Every prediction is the teacher-forced one (view k from ground-truth views 0..k-1).  Scenes
are drawn from the frozen view manifest with ``--seed`` unless named.  Runs headless: sheets are composed with Pillow;
``index.json`` lists what was written.
"""
from __future__ import annotations

import argparse
import json
import random
import re
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch

from .evaluate import AMP, MetricComputer, load_config, load_model
from .registry import DEFAULT_REGISTRY, load_registry, preflight
from .views import FixedViewDataset

HEADER, CAPTION = 72, 64


def safe_name(value: str) -> str:
    return re.sub(r"[^A-Za-z0-9._-]+", "_", str(value)).strip("_") or "unnamed"


def to_image(t: torch.Tensor):
    """[3, H, W] in [0, 1] -> PIL image."""
    from PIL import Image
    arr = (t.detach().float().clamp(0, 1).permute(1, 2, 0).cpu().numpy() * 255.0 + 0.5).astype(np.uint8)
    return Image.fromarray(arr)


def compose_grid(rows, pad: int = 2) -> np.ndarray:
    """rows: list of lists of [3, H, W] tensors in [0, 1] -> uint8 [H_total, W_total, 3] with white gutters."""
    h, w = rows[0][0].shape[-2:]
    out = np.full((len(rows) * (h + pad) + pad, len(rows[0]) * (w + pad) + pad, 3), 255, dtype=np.uint8)
    for r, row in enumerate(rows):
        for c, img in enumerate(row):
            y, x = pad + r * (h + pad), pad + c * (w + pad)
            out[y:y + h, x:x + w] = np.asarray(to_image(img))
    return out


def build_sheet(scene_id: str, views: Sequence[int], context: Dict[int, object], truth: Dict[int, object],
                predictions: Dict[str, Dict[int, object]], metrics: Dict[str, Dict[int, Dict[str, float]]]):
    from PIL import Image, ImageDraw
    labels = ["Latest GT context", "Ground truth", *predictions.keys()]
    tile_w, tile_h = context[views[0]].size
    sheet = Image.new("RGB", (tile_w * len(labels), HEADER + (tile_h + CAPTION) * len(views)), "white")
    draw = ImageDraw.Draw(sheet)
    draw.text((10, 7), f"Scene: {scene_id}", fill="black")
    draw.text((10, 29), "Teacher-forced sequential synthesis: target view k uses ground-truth views 0..k-1", fill="black")
    for col, label in enumerate(labels):
        width = draw.textlength(label)
        draw.text((col * tile_w + max((tile_w - width) // 2, 8), 51), label, fill="black")
    for row, k in enumerate(views):
        y = HEADER + row * (tile_h + CAPTION)
        sheet.paste(context[k], (0, y))
        sheet.paste(truth[k], (tile_w, y))
        draw.text((8, y + tile_h + 4), f"Latest: GT view {k - 1}\nFull context: GT views 0..{k - 1}", fill="black",
                  spacing=3)
        draw.text((tile_w + 8, y + tile_h + 4), f"Target: GT view {k}", fill="black")
        for col, (label, images) in enumerate(predictions.items(), start=2):
            sheet.paste(images[k], (col * tile_w, y))
            m = metrics[label][k]
            lp = "n/a" if m["lpips"] != m["lpips"] else f"{m['lpips']:.4f}"
            draw.text((col * tile_w + 6, y + tile_h + 4), f"PSNR {m['psnr']:.2f}   SSIM {m['ssim']:.4f}\nLPIPS {lp}",
                      fill="black", spacing=3)
    return sheet


@torch.no_grad()
def render(registry, dataset: str, experiments, out_root: Path, scene_ids=None, scene_count: int = 8,
           view_indices=(1, 12, 23), seed: int = 9595, device: str = "cpu", amp_dtype: str = "bf16",
           allow_missing_checkpoint: bool = False, lpips=None) -> List[str]:
    reg = load_registry(registry)
    exps = [reg[e] for e in experiments]
    for e in exps:
        if e.dataset != dataset:
            raise ValueError(f"{e.name} belongs to dataset {e.dataset}, not {dataset}")
        problems = preflight(e, require_checkpoint=not allow_missing_checkpoint)
        if problems:
            raise SystemExit("preflight failed:\n  " + "\n  ".join(problems))
    size = exps[0].image_size or int(load_config(exps[0])["model"]["image_size"])
    ds = FixedViewDataset(str(exps[0].view_manifest), size, dataset_manifest=str(exps[0].manifest))
    order = list(range(len(ds)))
    if scene_ids:
        wanted = set(scene_ids)
        order = [i for i in order if ds.scenes[i]["scene_id"] in wanted]
        missing = wanted - {ds.scenes[i]["scene_id"] for i in order}
        if missing:
            raise KeyError(f"scenes not in the view manifest: {sorted(missing)}")
    else:
        random.Random(seed).shuffle(order)
        order = order[:scene_count]
    views = [v for v in view_indices if 1 <= v < ds.num_views]
    if not views:
        raise ValueError(f"no view index in 1..{ds.num_views - 1} among {list(view_indices)}")
    samples = {}
    for i in order:
        item = ds[i]
        samples[item.pop("scene_id")] = item
    computer = MetricComputer(lpips)
    use_amp = str(device).startswith("cuda") and amp_dtype != "fp32"
    predictions: Dict[str, Dict[str, Dict[int, object]]] = {}
    metrics: Dict[str, Dict[str, Dict[int, Dict[str, float]]]] = {}
    for e in exps:                                       # one model in memory at a time
        label = e.display_name or e.name
        model, _ = load_model(e, device, allow_missing_checkpoint)
        predictions[label], metrics[label] = {}, {}
        for sid, item in samples.items():
            batch = {k: v[None].to(device) for k, v in item.items()}
            with torch.autocast("cuda", dtype=AMP[amp_dtype], enabled=use_amp):
                pred = model(batch)["rendering"][0].float()             # views 1..V-1
            chosen = torch.stack([pred[k - 1] for k in views])
            target = torch.stack([batch["image"][0, k] for k in views]).float()
            vals = {name: v.detach().cpu().tolist() for name, v in computer(target, chosen).items()}
            predictions[label][sid] = {k: to_image(chosen[j]) for j, k in enumerate(views)}
            metrics[label][sid] = {k: {name: float(vals[name][j]) for name in vals} for j, k in enumerate(views)}
        del model
        if str(device).startswith("cuda"):
            torch.cuda.empty_cache()
    out_root = Path(out_root) / dataset
    out_root.mkdir(parents=True, exist_ok=True)
    written = []
    for sid, item in samples.items():
        folder = out_root / safe_name(sid)
        folder.mkdir(parents=True, exist_ok=True)
        truth = {k: to_image(item["image"][k]) for k in views}
        context = {k: to_image(item["image"][k - 1]) for k in views}
        to_image(item["image"][0]).save(folder / "input_view_00.png")
        for k in views:
            truth[k].save(folder / f"ground_truth_view_{k:02d}.png")
            for label in predictions:
                predictions[label][sid][k].save(folder / f"{safe_name(label)}_view_{k:02d}.png")
        sheet = build_sheet(sid, views, context, truth, {lab: predictions[lab][sid] for lab in predictions},
                            {lab: metrics[lab][sid] for lab in metrics})
        sheet.save(folder / "comparison.png")
        written.append(str(folder / "comparison.png"))
    with open(out_root / "index.json", "w") as fh:
        json.dump({"dataset": dataset, "scene_ids": list(samples), "view_indices": views, "seed": seed,
                   "conditioning_protocol": "teacher_forced_sequential",
                   "models": [e.display_name or e.name for e in exps], "metrics": metrics, "files": written}, fh, indent=1)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Comparison sheets of several evaluated models on the same scenes.")
    ap.add_argument("--registry", type=Path, default=DEFAULT_REGISTRY)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--experiment", action="append", required=True)
    ap.add_argument("--scene-id", action="append")
    ap.add_argument("--scene-count", type=int, default=8)
    ap.add_argument("--view-indices", default="1,12,23")
    ap.add_argument("--seed", type=int, default=9595)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--amp-dtype", choices=tuple(AMP), default="bf16")
    ap.add_argument("--output-root", "--output-dir", dest="output_root", type=Path, required=True)
    ap.add_argument("--allow-missing-checkpoint", action="store_true")
    args = ap.parse_args(argv)
    views = tuple(int(v) for v in args.view_indices.split(","))
    lpips = None
    try:
        from ..perceptual import build_lpips
        lpips = build_lpips(args.device)
    except Exception as exc:
        print(f"LPIPS unavailable ({exc}); its figure is left out")
    files = render(args.registry, args.dataset, args.experiment, args.output_root, args.scene_id, args.scene_count,
                   views, args.seed, args.device, args.amp_dtype, args.allow_missing_checkpoint, lpips)
    print(f"Wrote {len(files)} comparison grids to {args.output_root / args.dataset}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
