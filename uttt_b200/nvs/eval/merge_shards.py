"""Merge the shards of one experiment into a single evaluation (uttt_nvs/eval/merge_sharded_evaluations.py).

    python -m uttt_b200.nvs.eval.merge_shards --registry R --experiment E --shards-root DIR --num-shards S \
        --output-root OUT [--overwrite]

Every shard must be complete; scenes must not repeat across shards; the merged row count is checked against the
registry's expected scene count when it is given.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from .evaluate import shard_dir, summarize
from .registry import load_registry


def merge(exp, shards_root: Path, num_shards: int, out_root: Path, bootstrap_samples: int = 10000,
          overwrite: bool = False, allow_incomplete: bool = False):
    rows, seen = [], set()
    for i in range(num_shards):
        d = shard_dir(shards_root, exp.name, i, num_shards)
        if not (d / "summary.json").exists():
            raise FileNotFoundError(f"shard {i} of {num_shards} is not finished: {d}")
        with open(d / "raw_metrics.jsonl") as fh:
            shard_rows = [json.loads(ln) for ln in fh if ln.strip()]
        shard_scenes = {r["scene_id"] for r in shard_rows}
        if seen & shard_scenes:
            raise ValueError(f"shard {i} repeats scenes of an earlier shard: {sorted(seen & shard_scenes)[:3]}")
        seen |= shard_scenes
        rows.extend(shard_rows)
    if exp.expected_scenes and len(seen) != int(exp.expected_scenes) and not allow_incomplete:
        raise ValueError(f"merged {len(seen)} scenes, the registry expects {exp.expected_scenes}")
    out_dir = shard_dir(out_root, exp.name, 0, 1)
    if (out_dir / "summary.json").exists() and not overwrite:
        raise FileExistsError(f"{out_dir} already holds a merged evaluation")
    out_dir.mkdir(parents=True, exist_ok=True)
    rows.sort(key=lambda r: (r["scene_id"], r["view"]))
    with open(out_dir / "raw_metrics.jsonl", "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    per_scene, summary = summarize(rows, bootstrap_samples)
    summary.update({"experiment": exp.name, "dataset": exp.dataset, "paper_model": exp.paper_model,
                    "display_name": exp.display_name, "merged_from_shards": num_shards})
    with open(out_dir / "scene_metrics.json", "w") as fh:
        json.dump(per_scene, fh, indent=1, sort_keys=True)
    with open(out_dir / "summary.json", "w") as fh:
        json.dump(summary, fh, indent=1, sort_keys=True)
    return summary


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--registry", type=Path, required=True)
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--shards-root", type=Path, required=True)
    ap.add_argument("--num-shards", type=int, required=True)
    ap.add_argument("--output-root", type=Path, required=True)
    ap.add_argument("--bootstrap-samples", type=int, default=10_000)
    ap.add_argument("--allow-incomplete", action="store_true")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    exp = load_registry(args.registry)[args.experiment]
    print(json.dumps(merge(exp, args.shards_root, args.num_shards, args.output_root, args.bootstrap_samples,
                           args.overwrite, args.allow_incomplete), sort_keys=True))


if __name__ == "__main__":
    main()
