"""Full-test evaluation of one registry entry (uttt_nvs/eval/evaluate.py).

    python -m uttt_b200.nvs.eval.evaluate --experiment gso_uttt_moe_e32a2 [--registry experiments.yaml] \
        [--output-root DIR] [--max-scenes N] [--shard-index I --num-shards S] [--device cuda:0] \
        [--amp-dtype bf16] [--bootstrap-samples 10000] [--wandb-mode disabled|offline|online] [--overwrite] \
        [--allow-missing-checkpoint]

Protocol ("nvs-eval-v2"): 24 ordered views per scene from the frozen view manifest; the forward pass is
teacher-forced sequential synthesis (the prediction of view k is conditioned on ground-truth views 0..k-1); view 0
only conditions; views 1..23 are scored with PSNR, SSIM and LPIPS-VGG (NaN when the perceptual weights are absent).

Artefacts, in ``<output-root>/<dataset>/<id>/`` with the reference's names and columns so that results of both
implementations merge, aggregate and plot together:

* ``raw_metrics.csv`` (``dataset, model, scene_id, view_index, psnr, ssim, lpips``; written row by row into
  ``raw_metrics.partial.csv`` while the run is going), ``raw_metrics.parquet`` when pyarrow is present;
* ``per_view_summary.csv``, ``overall_summary.json`` (scene-macro means with scene-bootstrap 95 % intervals);
* ``run_metadata.json`` (registry entry, digests of checkpoint / config / manifests / registry / evaluator sources,
  deterministic runtime fingerprint, run signature);
* ``completion.json``, written last: a folder without it is an interrupted run and is recomputed.

A scene shard ``i`` of ``S`` takes scenes ``i, i+S, ...``; run it with ``--output-root <shards>/shard_<i>`` and merge
with :mod:`uttt_b200.nvs.eval.merge_shards`.  ``--max-scenes`` without ``--output-root`` writes to
``eval_outputs_smoke/n<N>/`` beside the registry's output root, never into the full results.
"""
from __future__ import annotations

import argparse
import csv
import json
import time
from pathlib import Path
from typing import Any, Dict, Optional

import torch
import yaml

from .. import metrics as M
from ..model import resolve_model_class
from ..trainer import apply_overrides
from . import stats
from .fingerprint import (canonical_json_sha256, deterministic_runtime_fingerprint, evaluation_code_sha256, file_sha256,
                          git_commit, runtime_fingerprint_sha256)
from .registry import (DEFAULT_REGISTRY, Experiment, experiment_dir, output_root, preflight, resolve_experiment,
                       validate_v_gap)
from .views import FixedViewDataset

AMP = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
PROTOCOL = "nvs-eval-v2"
CONDITIONING = "teacher_forced_sequential"


def run_signature(experiment_id: str, assets: Dict[str, Any], runtime: Dict[str, Any], amp_dtype: str) -> str:
    """Identity of an evaluation: what was scored (asset digests), on what runtime, under which protocol."""
    return canonical_json_sha256({"protocol_version": PROTOCOL, "experiment_id": experiment_id, "assets": dict(assets),
                                  "runtime": dict(runtime), "amp_dtype": amp_dtype,
                                  "conditioning_protocol": CONDITIONING})


def load_config(exp: Experiment) -> Dict[str, Any]:
    with open(exp.config) as fh:
        cfg = yaml.safe_load(fh)
    if exp.overrides:
        cfg = apply_overrides(cfg, exp.overrides)
    return cfg


def load_model(exp: Experiment, device, allow_missing_checkpoint: bool = False, cfg: Optional[Dict[str, Any]] = None):
    """The model of the entry's configuration with the entry's checkpoint loaded strictly: a missing or an
    unexpected tensor is an error (wrapper prefixes of DDP / activation checkpointing / compilation are stripped)."""
    cfg = cfg or load_config(exp)
    model = resolve_model_class(cfg["model"].get("class_name"))(cfg)
    info: Dict[str, Any] = {"fwdbwd_pass_step": None, "param_update_step": None}
    if exp.checkpoint is not None and exp.checkpoint.is_file():
        ckpt = torch.load(exp.checkpoint, map_location="cpu", weights_only=False)
        if not isinstance(ckpt, dict) or "model" not in ckpt:
            raise ValueError(f"Unsupported checkpoint format: {exp.checkpoint}")
        from ..checkpoint import clean_key
        model.load_state_dict({clean_key(k): v for k, v in ckpt["model"].items()}, strict=True)
        info = {"fwdbwd_pass_step": ckpt.get("fwdbwd_pass_step"), "param_update_step": ckpt.get("param_update_step")}
    elif not allow_missing_checkpoint:
        raise FileNotFoundError(f"checkpoint not found: {exp.checkpoint}")
    return model.to(device).eval(), info


class MetricComputer:
    """PSNR / SSIM / LPIPS per image for [n, 3, H, W] batches in [0, 1]; LPIPS in chunks of ``lpips_batch_size``."""

    def __init__(self, lpips=None, lpips_batch_size: int = 32):
        if lpips_batch_size <= 0:
            raise ValueError("lpips_batch_size must be positive")
        self.lpips, self.chunk = lpips, lpips_batch_size

    @torch.no_grad()
    def __call__(self, target: torch.Tensor, pred: torch.Tensor) -> Dict[str, torch.Tensor]:
        if target.ndim != 4 or pred.ndim != 4:
            raise ValueError("metric inputs must both be NCHW tensors")
        if target.shape != pred.shape:
            raise ValueError(f"metric input shapes differ: {tuple(target.shape)} vs {tuple(pred.shape)}")
        target, pred = target.float().clamp(0, 1), pred.float().clamp(0, 1)
        out = {"psnr": M.psnr(pred, target), "ssim": M.ssim(pred, target)}
        if self.lpips is None:
            out["lpips"] = torch.full_like(out["psnr"], float("nan"))
        else:
            out["lpips"] = torch.cat([self.lpips(pred[i:i + self.chunk], target[i:i + self.chunk]).reshape(-1)
                                      for i in range(0, pred.shape[0], self.chunk)])
        return out


class Tracker:
    """Optional Weights & Biases run (``--wandb-mode offline|online``); ``disabled`` needs no package."""

    def __init__(self, mode: str, exp: Experiment, metadata: Dict[str, Any], max_scenes, out_dir: Path):
        self.run, self.id = None, None
        if mode == "disabled":
            return
        try:
            import wandb
        except ImportError as exc:
            raise RuntimeError("--wandb-mode offline/online needs the wandb package; use --wandb-mode disabled") from exc
        conf = exp.defaults.get("wandb", {}) or {}
        identity = {k: metadata.get(k) for k in ("experiment_id", "checkpoint_sha256", "config_sha256",
                                                 "view_manifest_sha256", "evaluation_code_sha256", "shard_index",
                                                 "num_shards")}
        identity.update(protocol=PROTOCOL, max_scenes=max_scenes)
        name = str(exp.raw.get("display_name", exp.name))
        if max_scenes is not None:
            name += f"-smoke-{max_scenes}"
        if (metadata.get("num_shards") or 1) > 1 and metadata.get("shard_index") is not None:
            name += f"-shard-{metadata['shard_index'] + 1:02d}-of-{metadata['num_shards']:02d}"
        tags = [exp.dataset, str(exp.raw.get("group", "")),
                f"v_gap-{'null' if metadata.get('v_gap') is None else metadata['v_gap']}",
                str(exp.raw.get("evaluation_class", "formal"))] + (["legacy"] if exp.raw.get("legacy") else [])
        self.run = wandb.init(entity=conf.get("entity"), project=conf.get("project", "nvs-eval"), name=name,
                              group=exp.dataset, job_type="full-test-metrics",
                              id=canonical_json_sha256(identity)[:12], resume="allow", mode=mode,
                              dir=str(out_dir / "wandb"), config=metadata, tags=tags)
        self.id = self.run.id

    def log(self, payload):
        if self.run is not None:
            self.run.log(payload)

    def summary(self, **kv):
        if self.run is not None:
            for k, v in kv.items():
                self.run.summary[k] = v

    def finish(self):
        if self.run is not None:
            self.run.finish()


def evaluate_experiment(exp: Experiment, out_dir: Path, registry_path: Optional[Path] = None, device: str = "cpu",
                        amp_dtype: str = "bf16", batch_size: int = 1, num_workers: int = 0, shard_index: int = 0,
                        num_shards: int = 1, max_scenes: Optional[int] = None, bootstrap_samples: int = 10_000,
                        allow_missing_checkpoint: bool = False, progress_every: int = 10, lpips=None,
                        lpips_batch_size: int = 32, wandb_mode: str = "disabled", image_workers: int = 8):
    """Scores the entry and writes every artefact; returns the overall summary."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    partial, completion = out_dir / "raw_metrics.partial.csv", out_dir / "completion.json"
    cfg = load_config(exp)
    v_gap = validate_v_gap(exp, cfg)
    image_size = exp.image_size or int(cfg["model"]["image_size"])
    ds = FixedViewDataset(str(exp.view_manifest), image_size, shard_index, num_shards, max_scenes or 0,
                          dataset_manifest=str(exp.manifest), expected_num_views=exp.num_views,
                          load_threads=image_workers)
    scored = exp.scored_views
    loader = torch.utils.data.DataLoader(ds, batch_size=batch_size, num_workers=num_workers, shuffle=False,
                                         pin_memory=str(device).startswith("cuda"), drop_last=False,
                                         persistent_workers=num_workers > 0)
    model, ckpt_info = load_model(exp, device, allow_missing_checkpoint, cfg)
    computer = MetricComputer(lpips, lpips_batch_size)

    have_ckpt = exp.checkpoint is not None and exp.checkpoint.is_file()
    assets = {"registry_sha256": file_sha256(registry_path) if registry_path else None,
              "checkpoint_sha256": file_sha256(exp.checkpoint) if have_ckpt else None,
              "config_sha256": file_sha256(exp.config), "dataset_manifest_sha256": file_sha256(exp.manifest),
              "view_manifest_sha256": file_sha256(exp.view_manifest), "code_commit": git_commit(),
              "evaluation_code_sha256": evaluation_code_sha256()}
    runtime = deterministic_runtime_fingerprint(device)
    display = str(exp.raw.get("display_name", exp.model_name))
    metadata = {
        "protocol_version": PROTOCOL, "run_signature": run_signature(exp.name, assets, runtime, amp_dtype),
        "experiment_id": exp.name, "dataset": exp.dataset, "model": display, "paper_model": exp.model_name,
        "checkpoint_impl": exp.raw.get("checkpoint_impl"), "checkpoint": str(exp.checkpoint),
        "checkpoint_step": exp.raw.get("checkpoint_step"), "config": str(exp.config),
        "dataset_manifest": str(exp.manifest), "view_manifest": str(exp.view_manifest),
        "registry": str(registry_path) if registry_path else None, **assets,
        "runtime": runtime, "runtime_sha256": runtime_fingerprint_sha256(runtime), "assets": assets, "v_gap": v_gap,
        "evaluation_class": exp.raw.get("evaluation_class", "formal"),
        "source_wandb_run": exp.raw.get("source_wandb_run"), "source_commit": exp.raw.get("source_commit"),
        "num_views": exp.num_views, "scored_views": list(range(1, exp.num_views)),
        "conditioning_protocol": CONDITIONING,
        "conditioning_definition": "prediction for View k is conditioned on ground-truth Views 0..k-1",
        "amp_dtype": amp_dtype, "max_scenes": max_scenes, "shard_index": shard_index, "num_shards": num_shards,
        "lpips_available": lpips is not None, "implementation": "uttt_b200", **ckpt_info}
    (out_dir / "run_metadata.json").write_text(json.dumps(metadata, indent=2, sort_keys=True, default=str) + "\n",
                                               encoding="utf-8")
    tracker = Tracker(wandb_mode, exp, metadata, max_scenes, out_dir)
    records = []
    t0 = time.time()
    use_amp = str(device).startswith("cuda") and amp_dtype != "fp32"
    try:
        with open(partial, "w", newline="", encoding="utf-8") as fh:
            writer = csv.DictWriter(fh, fieldnames=stats.RAW_FIELDS)
            writer.writeheader()
            with torch.inference_mode():
                for i, batch in enumerate(loader):
                    sids = batch.pop("scene_id")
                    sids = [sids] if isinstance(sids, str) else [str(s) for s in sids]
                    batch = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
                    with torch.autocast("cuda", dtype=AMP[amp_dtype], enabled=use_amp):
                        out = model(batch)
                    pred, tgt = out["rendering"].float(), out["target"]["image"].float()       # [b, V-1, 3, H, W]
                    if pred.shape[1] != scored or tgt.shape[1] != scored:
                        raise RuntimeError(f"model must produce exactly View 1..{scored}; got target "
                                           f"{tuple(tgt.shape)} and prediction {tuple(pred.shape)}")
                    vals = {k: v.detach().cpu().tolist()
                            for k, v in computer(tgt.flatten(0, 1), pred.flatten(0, 1)).items()}
                    for b, sid in enumerate(sids):
                        for v in range(1, scored + 1):
                            j = b * scored + v - 1
                            rec = {"dataset": exp.dataset, "model": display, "scene_id": sid, "view_index": v,
                                   "psnr": float(vals["psnr"][j]), "ssim": float(vals["ssim"][j]),
                                   "lpips": float(vals["lpips"][j])}
                            writer.writerow(rec)
                            records.append(rec)
                    fh.flush()
                    if i % max(progress_every, 1) == 0 or i + 1 == len(loader):
                        tracker.log({"progress/scenes": len(records) // scored, "progress/batches": i + 1})
                        print(f"[{exp.name}] {i + 1}/{len(loader)} batches, {time.time() - t0:.0f}s", flush=True)
        n_scenes = len(ds)
        stats.validate_complete(records, n_scenes, n_scenes * scored, scored)
        if max_scenes is None and num_shards == 1 and exp.expected_scenes is not None:
            if n_scenes != exp.expected_scenes:
                raise RuntimeError(f"registry expects {exp.expected_scenes} scenes, dataset contains {n_scenes}")
            if exp.expected_rows is not None and n_scenes * scored != exp.expected_rows:
                raise RuntimeError(f"registry expects {exp.expected_rows} rows, evaluation produced "
                                   f"{n_scenes * scored}")
        overall, _ = stats.write_evaluation_outputs(records, out_dir, bootstrap_samples, exp.bootstrap_seed, scored)
        overall.update(runtime_seconds=time.time() - t0, expected_scenes=n_scenes, expected_rows=n_scenes * scored)
        (out_dir / "overall_summary.json").write_text(json.dumps(overall, indent=2, sort_keys=True) + "\n",
                                                      encoding="utf-8")
        tracker.summary(**overall, state="complete")
        partial.unlink(missing_ok=True)
        digests = {n: file_sha256(out_dir / n)
                   for n in ("raw_metrics.csv", "raw_metrics.parquet", "overall_summary.json", "per_view_summary.csv",
                             "run_metadata.json") if (out_dir / n).is_file()}
        payload = {"state": "complete", "experiment_id": exp.name, "dataset": exp.dataset,
                   "expected_scenes": n_scenes, "expected_rows": n_scenes * scored,
                   "run_signature": metadata["run_signature"], "runtime_sha256": metadata["runtime_sha256"],
                   **{k: assets[k] for k in ("registry_sha256", "dataset_manifest_sha256", "checkpoint_sha256",
                                             "config_sha256", "view_manifest_sha256", "evaluation_code_sha256")},
                   "raw_metrics_sha256": digests["raw_metrics.csv"], "artifact_sha256": digests,
                   "wandb_run_id": tracker.id, "wandb_mode": wandb_mode}
    except Exception:
        tracker.summary(state="failed", partial_rows=len(records))
        raise
    finally:
        tracker.finish()
    tmp = completion.with_suffix(".json.tmp")
    tmp.write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    tmp.replace(completion)
    return overall


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Full-test evaluation of one registry entry.")
    ap.add_argument("--registry", type=Path, default=DEFAULT_REGISTRY)
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--output-root", type=Path)
    ap.add_argument("--max-scenes", type=int)
    ap.add_argument("--shard-index", type=int, default=0)
    ap.add_argument("--num-shards", type=int, default=1)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--num-workers", type=int, default=0)
    ap.add_argument("--image-workers", type=int, default=8)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--amp-dtype", choices=tuple(AMP), default="bf16")
    ap.add_argument("--lpips-batch-size", type=int, default=32)
    ap.add_argument("--bootstrap-samples", type=int, default=10_000)
    ap.add_argument("--progress-every", type=int, default=10)
    ap.add_argument("--wandb-mode", choices=("online", "offline", "disabled"), default="disabled")
    ap.add_argument("--allow-missing-checkpoint", action="store_true",
                    help="score the randomly initialised model (pipeline checks only)")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    if args.batch_size <= 0:
        ap.error("--batch-size must be positive")
    if args.max_scenes is not None and args.max_scenes <= 0:
        ap.error("--max-scenes must be positive")
    if args.num_shards <= 0 or not 0 <= args.shard_index < args.num_shards:
        ap.error("--shard-index must satisfy 0 <= index < --num-shards")
    try:
        exp = resolve_experiment(args.registry, args.experiment)
    except KeyError as exc:
        raise SystemExit(str(exc))
    root = output_root(args.registry, args.output_root)
    if args.max_scenes is not None and args.output_root is None:
        root = root.parent / "eval_outputs_smoke" / f"n{args.max_scenes}"
    problems = preflight(exp, require_checkpoint=not args.allow_missing_checkpoint)
    if problems:
        raise SystemExit("Required evaluation inputs are missing:\n  - " + "\n  - ".join(problems))
    out_dir = experiment_dir(root, exp)
    completion = out_dir / "completion.json"
    if completion.exists() and not args.overwrite:
        raise SystemExit(f"{completion} marks this evaluation complete; pass --overwrite to rerun")
    if args.overwrite:
        completion.unlink(missing_ok=True)
    elif (out_dir / "raw_metrics.csv").exists():
        print(f"{out_dir / 'raw_metrics.csv'} exists without a completion marker; recomputing the interrupted run")
    if str(args.device).startswith("cuda") and not torch.cuda.is_available():
        raise SystemExit("CUDA was requested but is not available")
    lpips = None
    try:
        from ..perceptual import build_lpips
        lpips = build_lpips(args.device)
    except Exception as exc:      # the weights cannot be downloaded: they are read from files when given
        print(f"LPIPS unavailable ({exc}); its column is left empty")
    overall = evaluate_experiment(exp, out_dir, args.registry.resolve(), args.device, args.amp_dtype, args.batch_size,
                                  args.num_workers, args.shard_index, args.num_shards, args.max_scenes,
                                  args.bootstrap_samples, args.allow_missing_checkpoint, args.progress_every, lpips,
                                  args.lpips_batch_size, args.wandb_mode, args.image_workers)
    print(json.dumps({"experiment": exp.name, "output_dir": str(out_dir), "overall": overall}, indent=2, sort_keys=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
