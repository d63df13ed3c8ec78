"""Tables over finished evaluations (uttt_nvs/eval/aggregate.py).

    python -m uttt_b200.nvs.eval.aggregate [--registry R] [--output-root DIR] [--dataset gso] [--allow-incomplete]

Reads ``raw_metrics.csv``, ``per_view_summary.csv`` and ``overall_summary.json`` of every registry entry under
``<output-root>/<dataset>/<id>/`` and checks each raw table (column order, expected rows and scenes, every scored
view present).  Writes, in ``<output-root>/aggregate/``: ``all_overall_metrics.csv`` (one row per run),
``all_per_view_metrics.csv``, ``all_raw_metrics.parquet`` (when pyarrow is present; ``all_raw_metrics.csv``
otherwise), ``missing_runs.json``, and one Markdown table per dataset.  A missing run is an error unless
``--allow-incomplete``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from . import stats
from .registry import DEFAULT_REGISTRY, experiment_dir, load_registry, output_root


def aggregate(registry_path, out_root: Path, datasets=None, allow_incomplete: bool = False):
    reg = load_registry(registry_path)
    out_root = Path(out_root)
    agg = out_root / "aggregate"
    agg.mkdir(parents=True, exist_ok=True)
    wanted = set(datasets or [])
    raw_all, per_view_all, overall_all, missing = [], [], [], []
    for exp in reg.values():
        if wanted and exp.dataset not in wanted:
            continue
        d = experiment_dir(out_root, exp)
        need = {"raw": d / "raw_metrics.csv", "per_view": d / "per_view_summary.csv", "overall": d / "overall_summary.json"}
        absent = [str(p) for p in need.values() if not p.is_file()]
        if absent:
            missing.append({"experiment": exp.name, "files": absent})
            continue
        raw = stats.read_raw_csv(need["raw"])                       # raises on a different column order
        if exp.expected_rows is not None and len(raw) != exp.expected_rows:
            raise RuntimeError(f"{exp.name}: expected {exp.expected_rows} raw rows, got {len(raw)}")
        n_scenes = len({r["scene_id"] for r in raw})
        if exp.expected_scenes is not None and n_scenes != exp.expected_scenes:
            raise RuntimeError(f"{exp.name}: expected {exp.expected_scenes} scenes, got {n_scenes}")
        if {r["view_index"] for r in raw} != set(range(1, exp.num_views)):
            raise RuntimeError(f"{exp.name}: raw records do not cover View 1..{exp.num_views - 1}")
        raw_all.extend({"experiment_id": exp.name, **r} for r in raw)
        per_view_all.extend({"experiment_id": exp.name, **r} for r in stats.read_csv(need["per_view"]))
        overall = json.loads(need["overall"].read_text())
        overall_all.append({"experiment_id": exp.name, "dataset": exp.dataset, "model": exp.display_name,
                            "paper_model": exp.paper_model, "checkpoint_impl": exp.checkpoint_impl, **overall,
                            "dataset": exp.dataset, "model": exp.display_name})
    if missing and not allow_incomplete:
        raise FileNotFoundError(f"{len(missing)} registered evaluations are incomplete:\n"
                                + json.dumps(missing[:5], indent=2))
    if not raw_all:
        raise RuntimeError("No complete evaluation outputs were found")
    raw_fields = ("experiment_id",) + stats.RAW_FIELDS
    if not stats.write_parquet(agg / "all_raw_metrics.parquet", raw_fields, raw_all):
        stats.write_csv(agg / "all_raw_metrics.csv", raw_fields, raw_all)
    stats.write_csv(agg / "all_per_view_metrics.csv", ("experiment_id",) + stats.PER_VIEW_FIELDS, per_view_all)
    fields = []
    for row in overall_all:
        fields.extend(k for k in row if k not in fields)
    stats.write_csv(agg / "all_overall_metrics.csv", fields, overall_all)
    (agg / "missing_runs.json").write_text(json.dumps(missing, indent=2) + "\n", encoding="utf-8")
    for ds in sorted({r["dataset"] for r in overall_all}):
        lines = ["| model | PSNR | SSIM | LPIPS | scenes |", "|---|---|---|---|---|"]
        for r in overall_all:
            if r["dataset"] != ds:
                continue
            cells = []
            for m in stats.METRIC_NAMES:
                v, lo, hi = r.get(f"overall_{m}"), r.get(f"overall_{m}_ci95_low"), r.get(f"overall_{m}_ci95_high")
                cells.append("-" if v is None else f"{v:.3f} [{lo:.3f}, {hi:.3f}]")
            lines.append(f"| {r['model']} | " + " | ".join(cells) + f" | {r['num_valid_scenes']} |")
        (agg / f"table_{ds}.md").write_text("\n".join(lines) + "\n", encoding="utf-8")
    return {"runs": len(overall_all), "raw_rows": len(raw_all), "per_view_rows": len(per_view_all),
            "missing": len(missing), "dir": str(agg)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Validate and combine completed evaluation outputs.")
    ap.add_argument("--registry", type=Path, default=DEFAULT_REGISTRY)
    ap.add_argument("--output-root", type=Path)
    ap.add_argument("--dataset", action="append")
    ap.add_argument("--allow-incomplete", action="store_true")
    args = ap.parse_args(argv)
    out = aggregate(args.registry, output_root(args.registry, args.output_root), args.dataset, args.allow_incomplete)
    print(f"Aggregated {out['runs']} runs, {out['raw_rows']} raw rows, and {out['per_view_rows']} per-view summary "
          f"rows into {out['dir']}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
