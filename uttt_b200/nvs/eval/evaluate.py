"""Full-test evaluation of one registry entry (uttt_nvs/eval/evaluate.py).

    python -m uttt_b200.nvs.eval.evaluate --registry experiments.yaml --experiment gso/uttt_moe_e32a2 \
        [--output-root DIR] [--max-scenes N] [--shard-index I --num-shards S] [--device cuda:0] \
        [--amp-dtype bf16] [--bootstrap-samples 10000] [--allow-missing-checkpoint] [--overwrite]

Protocol: 24 ordered views per scene from the frozen view manifest; the forward pass is teacher-forced
sequential synthesis (the prediction of view k is conditioned on ground-truth views 0..k-1); view 0 only
conditions; views 1.. are scored with PSNR, SSIM and, when a perceptual network is available, LPIPS.
Outputs under ``<output-root>/<experiment>/``: ``raw_metrics.jsonl`` (one row per scene and view),
``scene_metrics.json``, ``summary.json`` (means with scene-bootstrap confidence intervals),
``run_metadata.json`` (registry entry + runtime fingerprint).
"""
from __future__ import annotations

import argparse
import json
import os
import time
from pathlib import Path

import torch
import yaml

from .. import metrics as M
from ..model import LVSMModel
from ..trainer import apply_overrides
from .fingerprint import file_sha256, runtime_fingerprint
from .registry import load_registry, output_root, preflight
from .views import FixedViewDataset

AMP = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


def shard_dir(root: Path, experiment: str, shard_index: int, num_shards: int) -> Path:
    base = root / experiment.replace("/", "__")
    return base if num_shards == 1 else base / f"shard_{shard_index:03d}_of_{num_shards:03d}"


def summarize(rows, bootstrap_samples: int, seed: int = 9595):
    """rows: dicts with scene_id, view, psnr, ssim[, lpips] -> per-scene means and bootstrap CIs over scenes."""
    scenes = {}
    for r in rows:
        scenes.setdefault(r["scene_id"], []).append(r)
    per_scene = {}
    keys = [k for k in ("psnr", "ssim", "lpips") if rows and k in rows[0] and rows[0][k] is not None]
    for sid, rs in scenes.items():
        per_scene[sid] = {k: sum(r[k] for r in rs) / len(rs) for k in keys}
        per_scene[sid]["views"] = len(rs)
    summary = {"num_scenes": len(scenes), "num_rows": len(rows)}
    for k in keys:
        vals = [per_scene[s][k] for s in sorted(per_scene)]
        ci = M.bootstrap_ci(vals, resamples=bootstrap_samples, seed=seed)
        summary[k] = {"mean": ci["mean"], "ci95": [ci["ci_low"], ci["ci_high"]]}
    return per_scene, summary


def load_model(exp, device, allow_missing_checkpoint: bool):
    with open(exp.config) as fh:
        cfg = yaml.safe_load(fh)
    if exp.overrides:
        cfg = apply_overrides(cfg, exp.overrides)
    model = LVSMModel(cfg)
    info = {"checkpoint": None}
    if exp.checkpoint is not None and exp.checkpoint.is_file():
        sd = torch.load(exp.checkpoint, map_location="cpu", weights_only=False)
        sd = sd.get("model", sd)
        from ..checkpoint import clean_key
        missing, unexpected = model.load_state_dict({clean_key(k): v for k, v in sd.items()}, strict=False)
        info = {"checkpoint": str(exp.checkpoint), "checkpoint_sha256_head": file_sha256(exp.checkpoint, 64 << 20),
                "missing_keys": list(missing), "unexpected_keys": list(unexpected)}
    elif not allow_missing_checkpoint:
        raise FileNotFoundError(f"checkpoint not found: {exp.checkpoint}")
    return model.to(device).eval(), info


@torch.no_grad()
def evaluate_experiment(exp, out_dir: Path, device: str = "cpu", amp_dtype: str = "bf16", batch_size: int = 1,
                        num_workers: int = 0, shard_index: int = 0, num_shards: int = 1, max_scenes: int = 0,
                        bootstrap_samples: int = 10000, allow_missing_checkpoint: bool = False,
                        progress_every: int = 10, lpips=None):
    out_dir.mkdir(parents=True, exist_ok=True)
    model, ckpt_info = load_model(exp, device, allow_missing_checkpoint)
    ds = FixedViewDataset(str(exp.view_manifest), exp.image_size, shard_index, num_shards, max_scenes,
                          dataset_manifest=str(exp.manifest), expected_num_views=exp.num_views)
    loader = torch.utils.data.DataLoader(ds, batch_size=batch_size, num_workers=num_workers, shuffle=False)
    rows = []
    t0 = time.time()
    use_amp = device.startswith("cuda") and amp_dtype != "fp32"
    for i, batch in enumerate(loader):
        sids = batch.pop("scene_id")
        batch = {k: v.to(device) for k, v in batch.items()}
        with torch.autocast("cuda", dtype=AMP[amp_dtype], enabled=use_amp):
            out = model(batch)
        pred = out["rendering"].float().clamp(0, 1)          # [b, V-1, 3, H, W]: views 1..V-1
        tgt = out["target"].float()
        for b, sid in enumerate(sids):
            for v in range(pred.shape[1]):
                row = {"scene_id": sid, "view": v + 1, "psnr": float(M.psnr(pred[b, v], tgt[b, v])),
                       "ssim": float(M.ssim(pred[b, v][None], tgt[b, v][None])),
                       "lpips": None if lpips is None else float(lpips(pred[b, v][None], tgt[b, v][None]))}
                rows.append(row)
        if progress_every and (i + 1) % progress_every == 0:
            print(f"[{exp.name}] {i + 1}/{len(loader)} batches, {time.time() - t0:.0f}s", flush=True)
    with open(out_dir / "raw_metrics.jsonl", "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    per_scene, summary = summarize(rows, bootstrap_samples)
    summary.update({"experiment": exp.name, "dataset": exp.dataset, "paper_model": exp.paper_model,
                    "display_name": exp.display_name, "scored_views_per_scene": exp.scored_views,
                    "shard_index": shard_index, "num_shards": num_shards, "seconds": time.time() - t0})
    with open(out_dir / "scene_metrics.json", "w") as fh:
        json.dump(per_scene, fh, indent=1, sort_keys=True)
    with open(out_dir / "summary.json", "w") as fh:
        json.dump(summary, fh, indent=1, sort_keys=True)
    meta = {"registry_entry": exp.raw, "checkpoint_impl": exp.checkpoint_impl, **ckpt_info,
            "fingerprint": runtime_fingerprint(device=device)}
    with open(out_dir / "run_metadata.json", "w") as fh:
        json.dump(meta, fh, indent=1, sort_keys=True, default=str)
    return summary


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--registry", type=Path, required=True)
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--output-root", type=Path)
    ap.add_argument("--max-scenes", type=int, default=0)
    ap.add_argument("--shard-index", type=int, default=0)
    ap.add_argument("--num-shards", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--num-workers", type=int, default=0)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--amp-dtype", choices=tuple(AMP), default="bf16")
    ap.add_argument("--bootstrap-samples", type=int, default=10_000)
    ap.add_argument("--progress-every", type=int, default=10)
    ap.add_argument("--allow-missing-checkpoint", action="store_true",
                    help="score the randomly initialised model (pipeline checks only)")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    reg = load_registry(args.registry)
    if args.experiment not in reg:
        raise SystemExit(f"unknown experiment {args.experiment!r}; known: {sorted(reg)[:8]} ...")
    exp = reg[args.experiment]
    problems = preflight(exp, require_checkpoint=not args.allow_missing_checkpoint)
    if problems:
        raise SystemExit("preflight failed:\n  " + "\n  ".join(problems))
    out_dir = shard_dir(output_root(args.registry, args.output_root), exp.name, args.shard_index, args.num_shards)
    if (out_dir / "summary.json").exists() and not args.overwrite:
        raise SystemExit(f"{out_dir} already holds a finished evaluation (use --overwrite)")
    lpips = None
    try:
        from ..perceptual import build_lpips
        lpips = build_lpips(args.device)
    except Exception as exc:      # weights are optional
        print(f"LPIPS unavailable ({exc}); scoring PSNR / SSIM only")
    summary = evaluate_experiment(exp, out_dir, args.device, args.amp_dtype, args.batch_size, args.num_workers,
                                  args.shard_index, args.num_shards, args.max_scenes, args.bootstrap_samples,
                                  args.allow_missing_checkpoint, args.progress_every, lpips)
    print(json.dumps(summary, sort_keys=True))


if __name__ == "__main__":
    main()
