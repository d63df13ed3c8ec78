"""Tables over finished evaluations (uttt_nvs/eval/aggregate.py).

    python -m uttt_b200.nvs.eval.aggregate --registry R [--output-root DIR] [--dataset gso] [--allow-incomplete]

Writes ``<output-root>/aggregate_<dataset>.{json,md}``: one row per registry entry with mean and 95 % scene-bootstrap
interval for every metric.  Missing evaluations are an error unless ``--allow-incomplete``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from .evaluate import shard_dir
from .registry import load_registry, output_root


def aggregate(registry_path, out_root: Path, datasets=None, allow_incomplete: bool = False):
    reg = load_registry(registry_path)
    tables = {}
    for exp in reg.values():
        if datasets and exp.dataset not in datasets:
            continue
        path = shard_dir(out_root, exp.name, 0, 1) / "summary.json"
        if not path.exists():
            if allow_incomplete:
                continue
            raise FileNotFoundError(f"no finished evaluation for {exp.name}: {path}")
        with open(path) as fh:
            s = json.load(fh)
        if exp.expected_scenes and s["num_scenes"] != int(exp.expected_scenes) and not allow_incomplete:
            raise ValueError(f"{exp.name}: {s['num_scenes']} scenes scored, {exp.expected_scenes} expected")
        tables.setdefault(exp.dataset, []).append({"experiment": exp.name, "model": exp.display_name or exp.paper_model,
                                                   **{k: s[k] for k in ("psnr", "ssim", "lpips") if k in s},
                                                   "num_scenes": s["num_scenes"], "num_rows": s["num_rows"]})
    out_root.mkdir(parents=True, exist_ok=True)
    for ds, rows in tables.items():
        with open(out_root / f"aggregate_{ds}.json", "w") as fh:
            json.dump(rows, fh, indent=1)
        metrics = [m for m in ("psnr", "ssim", "lpips") if any(m in r for r in rows)]
        lines = ["| model | " + " | ".join(metrics) + " | scenes |", "|---|" + "---|" * (len(metrics) + 1)]
        for r in rows:
            cells = []
            for m in metrics:
                cells.append("-" if m not in r else f"{r[m]['mean']:.3f} [{r[m]['ci95'][0]:.3f}, {r[m]['ci95'][1]:.3f}]")
            lines.append(f"| {r['model']} | " + " | ".join(cells) + f" | {r['num_scenes']} |")
        (out_root / f"aggregate_{ds}.md").write_text("\n".join(lines) + "\n")
    return tables


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--registry", type=Path, required=True)
    ap.add_argument("--output-root", type=Path)
    ap.add_argument("--dataset", action="append")
    ap.add_argument("--allow-incomplete", action="store_true")
    args = ap.parse_args(argv)
    tables = aggregate(args.registry, output_root(args.registry, args.output_root), args.dataset, args.allow_incomplete)
    print(json.dumps({k: len(v) for k, v in tables.items()}))


if __name__ == "__main__":
    main()
