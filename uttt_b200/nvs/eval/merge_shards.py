"""Merge the scene shards of one experiment into a single evaluation (uttt_nvs/eval/merge_sharded_evaluations.py).

    python -m uttt_b200.nvs.eval.merge_shards --registry R --experiment E --shards-root DIR --num-shards S \
        --output-root OUT [--overwrite]

Shard ``i`` is expected in ``<shards-root>/shard_<i>/<dataset>/<id>/`` (what ``evaluate --shard-index i --num-shards S
--output-root <shards-root>/shard_<i>`` writes).  A shard counts only with its ``completion.json``; its metadata must
name the right shard index and count; all shards must agree on experiment, dataset, checkpoint / config / view
manifest / evaluator digests and attention gap; no (scene, view) pair may repeat; the merged table must cover the
registry's expected scenes and rows.  The summaries are recomputed from the merged rows (10 000 resamples) and a new
``completion.json`` closes the merged folder.
"""
from __future__ import annotations

import argparse
import json
import shutil
import time
from pathlib import Path

from . import stats
from .registry import experiment_dir, resolve_experiment

INVARIANT_KEYS = ("experiment_id", "dataset", "checkpoint_sha256", "config_sha256", "view_manifest_sha256",
                  "evaluation_code_sha256", "v_gap")


def merge(exp, shards_root: Path, num_shards: int, out_root: Path, bootstrap_samples: int = 10_000,
          overwrite: bool = False, wandb_mode: str = "disabled"):
    if num_shards <= 0:
        raise ValueError("--num-shards must be positive")
    out_dir = experiment_dir(out_root, exp)
    completion = out_dir / "completion.json"
    if completion.exists() and not overwrite:
        raise FileExistsError(f"{completion} already marks a complete merge")
    records, metas = [], []
    for i in range(num_shards):
        d = experiment_dir(Path(shards_root) / f"shard_{i}", exp)
        need = [d / "completion.json", d / "raw_metrics.csv", d / "run_metadata.json"]
        if not all(p.is_file() for p in need):
            raise FileNotFoundError(f"incomplete shard {i}: {d}")
        meta = json.loads(need[2].read_text(encoding="utf-8"))
        if meta.get("shard_index") != i:
            raise ValueError(f"{d}: wrong shard_index metadata")
        if meta.get("num_shards") != num_shards:
            raise ValueError(f"{d}: wrong num_shards metadata")
        metas.append(meta)
        records.extend(stats.read_raw_csv(need[1]))
    for meta in metas[1:]:
        differ = [k for k in INVARIANT_KEYS if meta.get(k) != metas[0].get(k)]
        if differ:
            raise ValueError(f"shards disagree on metadata: {differ}")
    keys = [(r["scene_id"], r["view_index"]) for r in records]
    if len(keys) != len(set(keys)):
        raise ValueError("duplicate scene/view records across shards")
    scored = exp.scored_views
    scenes = exp.expected_scenes if exp.expected_scenes is not None else len({k[0] for k in keys})
    rows = exp.expected_rows if exp.expected_rows is not None else scenes * scored
    stats.validate_complete(records, scenes, rows, scored)
    if overwrite:
        shutil.rmtree(out_dir, ignore_errors=True)
    out_dir.mkdir(parents=True, exist_ok=True)
    records.sort(key=lambda r: (r["scene_id"], r["view_index"]))
    t0 = time.time()
    overall, _ = stats.write_evaluation_outputs(records, out_dir, bootstrap_samples, exp.bootstrap_seed, scored)
    meta = dict(metas[0])
    meta.update(max_scenes=None, shard_index=None, num_shards=num_shards,
                merge_protocol="deterministic strided scene shards", merged_at_unix=time.time())
    (out_dir / "run_metadata.json").write_text(json.dumps(meta, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    overall.update(runtime_seconds=time.time() - t0, expected_scenes=scenes, expected_rows=rows)
    (out_dir / "overall_summary.json").write_text(json.dumps(overall, indent=2, sort_keys=True) + "\n",
                                                  encoding="utf-8")
    from .evaluate import Tracker
    tracker = Tracker(wandb_mode, exp, meta, None, out_dir)
    try:
        tracker.summary(**overall, state="complete")
    finally:
        tracker.finish()
    completion.write_text(json.dumps({
        "state": "complete", "experiment_id": exp.name, "dataset": exp.dataset, "expected_scenes": scenes,
        "expected_rows": rows, **{k: meta.get(k) for k in ("checkpoint_sha256", "config_sha256",
                                                          "view_manifest_sha256", "evaluation_code_sha256")},
        "wandb_run_id": tracker.id, "wandb_mode": wandb_mode}, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    return overall


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Validate and merge the scene shards of one evaluation.")
    ap.add_argument("--registry", type=Path, required=True)
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--shards-root", type=Path, required=True)
    ap.add_argument("--num-shards", type=int, required=True)
    ap.add_argument("--output-root", type=Path, required=True)
    ap.add_argument("--bootstrap-samples", type=int, default=10_000)
    ap.add_argument("--wandb-mode", choices=("online", "offline", "disabled"), default="disabled")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    exp = resolve_experiment(args.registry, args.experiment)
    overall = merge(exp, args.shards_root, args.num_shards, args.output_root, args.bootstrap_samples, args.overwrite,
                    args.wandb_mode)
    print(json.dumps({"experiment": exp.name, "overall": overall}, indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
