"""Side-by-side comparison grids of several registry entries (uttt_nvs/eval/render_comparison.py).

    python -m uttt_b200.nvs.eval.render_comparison --registry R --dataset gso --experiment A --experiment B \
        [--scene-id S ...] [--scene-count 8] [--view-indices 1,12,23] [--seed 9595] [--device cuda:0] \
        [--amp-dtype bf16] --output-dir DIR [--allow-missing-checkpoint]

For each chosen scene one PNG: rows = ground truth followed by one row per experiment, columns = the chosen
views.  Scenes are drawn from the frozen view manifest with ``--seed`` unless named.  Runs headless: images are
composed as arrays and written with Pillow.
"""
from __future__ import annotations

import argparse
import json
import random
from pathlib import Path

import numpy as np
import torch

from .evaluate import AMP, load_config, load_model
from .registry import load_registry, preflight
from .views import FixedViewDataset


def compose_grid(rows, pad: int = 2) -> np.ndarray:
    """rows: list of lists of [3, H, W] tensors in [0, 1] -> uint8 [H_total, W_total, 3] with white gutters."""
    h, w = rows[0][0].shape[-2:]
    out = np.full((len(rows) * (h + pad) + pad, len(rows[0]) * (w + pad) + pad, 3), 255, dtype=np.uint8)
    for r, row in enumerate(rows):
        for c, img in enumerate(row):
            arr = (img.detach().float().clamp(0, 1).permute(1, 2, 0).cpu().numpy() * 255.0 + 0.5).astype(np.uint8)
            y, x = pad + r * (h + pad), pad + c * (w + pad)
            out[y:y + h, x:x + w] = arr
    return out


@torch.no_grad()
def render(registry, dataset: str, experiments, out_dir: Path, scene_ids=None, scene_count: int = 8,
           view_indices=(1, 12, 23), seed: int = 9595, device: str = "cpu", amp_dtype: str = "bf16",
           allow_missing_checkpoint: bool = False):
    from PIL import Image
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
    else:
        random.Random(seed).shuffle(order)
        order = order[:scene_count]
    models = [load_model(e, device, allow_missing_checkpoint)[0] for e in exps]
    out_dir.mkdir(parents=True, exist_ok=True)
    written = []
    use_amp = device.startswith("cuda") and amp_dtype != "fp32"
    for i in order:
        item = ds[i]
        sid = item.pop("scene_id")
        batch = {k: v[None].to(device) for k, v in item.items()}
        cols = [v for v in view_indices if 1 <= v < batch["image"].shape[1]]
        rows = [[batch["image"][0, v] for v in cols]]
        for model in models:
            with torch.autocast("cuda", dtype=AMP[amp_dtype], enabled=use_amp):
                pred = model(batch)["rendering"][0]              # views 1..V-1
            rows.append([pred[v - 1] for v in cols])
        path = out_dir / f"{dataset}__{sid.replace('/', '__')}.png"
        Image.fromarray(compose_grid(rows)).save(path)
        written.append(str(path))
    with open(out_dir / f"{dataset}__index.json", "w") as fh:
        json.dump({"rows": ["ground truth"] + [e.display_name or e.name for e in exps], "views": list(view_indices),
                   "files": written}, fh, indent=1)
    return written


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--registry", type=Path, required=True)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--experiment", action="append", required=True)
    ap.add_argument("--scene-id", action="append")
    ap.add_argument("--scene-count", type=int, default=8)
    ap.add_argument("--view-indices", default="1,12,23")
    ap.add_argument("--seed", type=int, default=9595)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--amp-dtype", choices=tuple(AMP), default="bf16")
    ap.add_argument("--output-dir", type=Path, required=True)
    ap.add_argument("--allow-missing-checkpoint", action="store_true")
    args = ap.parse_args(argv)
    views = tuple(int(v) for v in args.view_indices.split(","))
    files = render(args.registry, args.dataset, args.experiment, args.output_dir, args.scene_id, args.scene_count,
                   views, args.seed, args.device, args.amp_dtype, args.allow_missing_checkpoint)
    print(f"wrote {len(files)} grids to {args.output_dir}")


if __name__ == "__main__":
    main()
