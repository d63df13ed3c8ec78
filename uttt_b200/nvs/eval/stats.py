"""Raw per-view records and their scene-bootstrap summaries (uttt_nvs/eval/statistics.py).

One record per scene and scored view: ``dataset, model, scene_id, view_index, psnr, ssim, lpips`` (``RAW_FIELDS``, in
this column order in ``raw_metrics.csv``).  Summaries:

* overall: per metric the mean over scenes of the scene's mean over views ("scene macro"), the number of scenes with a
  finite value, and a 95 % percentile-bootstrap interval over scenes;
* per view: per metric and view index the mean over scenes, its interval and the count.

The resampling protocol is the published one, so that intervals computed by either implementation from the same
records are identical: ``numpy.random.default_rng(seed)``, indices drawn as ``integers(0, n, size=(rows, n))`` in
chunks of 512 resamples, seed = ``bootstrap_seed + 100000 * metric_number`` for the overall interval and
``+ view_index`` for a view's; with equal scene sets two models therefore see the same resamples (paired).
No pandas is needed; the Parquet copy of the raw table is written when ``pyarrow`` is importable.
"""
from __future__ import annotations

import csv
import json
import math
from pathlib import Path
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np

RAW_FIELDS = ("dataset", "model", "scene_id", "view_index", "psnr", "ssim", "lpips")
METRIC_NAMES = ("psnr", "ssim", "lpips")
PER_VIEW_FIELDS = ("dataset", "model", "view_index", "metric", "mean", "ci95_low", "ci95_high", "n_valid")
_CHUNK = 512


def _number(v) -> float:
    if v is None or v == "":
        return math.nan
    try:
        return float(v)
    except (TypeError, ValueError):
        return math.nan


def clean_records(records: Iterable[Mapping[str, Any]], scored_views: int = 23) -> List[Dict[str, Any]]:
    """Records restricted to ``RAW_FIELDS`` with typed values; a missing column or a view index outside
    ``1..scored_views`` is an error; a metric that does not parse becomes NaN (it then counts as not valid)."""
    out = []
    bad_views = set()
    for r in records:
        missing = [f for f in RAW_FIELDS if f not in r]
        if missing:
            raise ValueError(f"raw metric records are missing columns: {missing}")
        v = int(r["view_index"])
        if not 1 <= v <= scored_views:
            bad_views.add(v)
        out.append({"dataset": str(r["dataset"]), "model": str(r["model"]), "scene_id": str(r["scene_id"]),
                    "view_index": v, **{m: _number(r[m]) for m in METRIC_NAMES}})
    if bad_views:
        raise ValueError(f"view_index must be in 1..{scored_views}, got {sorted(bad_views)}")
    return out


def bootstrap_mean_ci(values: Sequence[float], samples: int, seed: int) -> Tuple[Optional[float], Optional[float]]:
    x = np.asarray(values, dtype=np.float64)
    x = x[np.isfinite(x)]
    if x.size == 0:
        return None, None
    if x.size == 1 or samples <= 0:
        return float(x[0]), float(x[0])
    rng = np.random.default_rng(seed)
    means = np.empty(samples, dtype=np.float64)
    for lo in range(0, samples, _CHUNK):
        hi = min(lo + _CHUNK, samples)
        means[lo:hi] = x[rng.integers(0, x.size, size=(hi - lo, x.size))].mean(axis=1)
    low, high = np.quantile(means, [0.025, 0.975])
    return float(low), float(high)


def summarize_records(records: Iterable[Mapping[str, Any]], bootstrap_samples: int = 10_000,
                      bootstrap_seed: int = 9595, scored_views: int = 23):
    """(overall dictionary, per-view rows) of the records of ONE dataset and ONE model."""
    rows = clean_records(records, scored_views)
    datasets, models = {r["dataset"] for r in rows}, {r["model"] for r in rows}
    if len(datasets) != 1 or len(models) != 1:
        raise ValueError("summarize_records expects exactly one dataset and one model")
    dataset, model = next(iter(datasets)), next(iter(models))
    scenes = sorted({r["scene_id"] for r in rows})
    overall: Dict[str, Any] = {"dataset": dataset, "model": model, "num_valid_scenes": len(scenes),
                               "num_valid_samples": len(rows), "bootstrap_samples": int(bootstrap_samples),
                               "bootstrap_seed": int(bootstrap_seed)}
    per_view = []
    for k, metric in enumerate(METRIC_NAMES):
        by_scene: Dict[str, List[float]] = {s: [] for s in scenes}
        by_view: Dict[int, List[float]] = {v: [] for v in range(1, scored_views + 1)}
        for r in rows:
            by_scene[r["scene_id"]].append(r[metric])
            if math.isfinite(r[metric]):
                by_view[r["view_index"]].append(r[metric])
        # a scene's mean skips its NaN views; an infinite view makes the scene's mean infinite, which is dropped
        scene_means = []
        for s in scenes:
            vals = [v for v in by_scene[s] if not math.isnan(v)]
            if vals and math.isfinite(sum(vals)):
                scene_means.append(sum(vals) / len(vals))
        overall[f"overall_{metric}"] = float(np.mean(scene_means)) if scene_means else None
        overall[f"overall_{metric}_n_valid"] = len(scene_means)
        lo, hi = bootstrap_mean_ci(scene_means, bootstrap_samples, bootstrap_seed + k * 100_000)
        overall[f"overall_{metric}_ci95_low"], overall[f"overall_{metric}_ci95_high"] = lo, hi
        for v in range(1, scored_views + 1):
            vals = by_view[v]
            lo, hi = bootstrap_mean_ci(vals, bootstrap_samples, bootstrap_seed + k * 100_000 + v)
            per_view.append({"dataset": dataset, "model": model, "view_index": v, "metric": metric,
                             "mean": float(np.mean(vals)) if vals else None, "ci95_low": lo, "ci95_high": hi,
                             "n_valid": len(vals)})
    return overall, per_view


def _cell(v):
    if v is None or (isinstance(v, float) and math.isnan(v)):
        return ""
    return repr(v) if isinstance(v, float) else v


def write_csv(path: Path, fields: Sequence[str], rows: Iterable[Mapping[str, Any]]) -> None:
    with open(path, "w", newline="", encoding="utf-8") as fh:
        w = csv.writer(fh)
        w.writerow(fields)
        for r in rows:
            w.writerow([_cell(r.get(f)) for f in fields])


def read_raw_csv(path: Path) -> List[Dict[str, Any]]:
    with open(path, newline="", encoding="utf-8") as fh:
        reader = csv.DictReader(fh)
        if tuple(reader.fieldnames or ()) != RAW_FIELDS:
            raise ValueError(f"{path}: unexpected raw-metric fields {reader.fieldnames}")
        return [{"dataset": r["dataset"], "model": r["model"], "scene_id": r["scene_id"],
                 "view_index": int(r["view_index"]), **{m: _number(r[m]) for m in METRIC_NAMES}} for r in reader]


def read_csv(path: Path) -> List[Dict[str, str]]:
    with open(path, newline="", encoding="utf-8") as fh:
        return list(csv.DictReader(fh))


def write_parquet(path: Path, fields: Sequence[str], rows: Sequence[Mapping[str, Any]]) -> bool:
    try:
        import pyarrow as pa
        import pyarrow.parquet as pq
    except ImportError:
        return False
    pq.write_table(pa.table({f: [r.get(f) for r in rows] for f in fields}), path)
    return True


def validate_complete(records: Sequence[Mapping[str, Any]], expected_scenes: int, expected_rows: int,
                      scored_views: int = 23) -> None:
    """Every scene must carry every scored view exactly once, and the counts must be the expected ones."""
    seen: Dict[str, List[int]] = {}
    for r in records:
        seen.setdefault(str(r["scene_id"]), []).append(int(r["view_index"]))
    want = list(range(1, scored_views + 1))
    incomplete = {s: sorted(set(want) - set(v)) for s, v in seen.items() if sorted(v) != want}
    if incomplete:
        raise RuntimeError(f"incomplete per-scene view coverage: {dict(list(incomplete.items())[:5])}")
    if len(seen) != expected_scenes:
        raise RuntimeError(f"expected {expected_scenes} scenes, got {len(seen)}")
    if len(records) != expected_rows:
        raise RuntimeError(f"expected {expected_rows} rows, got {len(records)}")


def write_evaluation_outputs(records: Iterable[Mapping[str, Any]], output_dir, bootstrap_samples: int = 10_000,
                             bootstrap_seed: int = 9595, scored_views: int = 23):
    """``raw_metrics.csv`` (+ ``raw_metrics.parquet``), ``per_view_summary.csv``, ``overall_summary.json``."""
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    rows = clean_records(records, scored_views)
    overall, per_view = summarize_records(rows, bootstrap_samples, bootstrap_seed, scored_views)
    write_csv(out / "raw_metrics.csv", RAW_FIELDS, rows)
    write_parquet(out / "raw_metrics.parquet", RAW_FIELDS, rows)
    write_csv(out / "per_view_summary.csv", PER_VIEW_FIELDS, per_view)
    (out / "overall_summary.json").write_text(json.dumps(overall, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    return overall, per_view
