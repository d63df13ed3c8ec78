"""Experiment registry of the full-test evaluation (uttt_nvs/eval/common.py, experiments.yaml).

A registry is a YAML file::

    defaults:
      checkpoint_root: /PATH/TO/CHECKPOINTS
      output_root: eval_outputs
      num_views: 24
      view_seed: 9595
    datasets:
      gso:   {manifest: /PATH/gso_local.txt, view_manifest: /PATH/gso_views.json, image_size: 256, num_scenes: 1019}
      dl3dv: {...}
    experiments:
      - name: gso/uttt_moe_e32a2
        dataset: gso
        config: configs/nvs/...yaml          # relative to the repository root
        checkpoint: gso/uttt_moe_e32a2/ckpt_0000000000024476.pt   # relative to checkpoint_root
        paper_model: uTTT-MoE-e32a2
        display_name: uTTT-MoE (32 experts, top-2)
        checkpoint_impl: uttt_moe
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import yaml

REPO_ROOT = Path(__file__).resolve().parents[3]
DEFAULT_NUM_VIEWS = 24
DEFAULT_VIEW_SEED = 9595


@dataclass
class Experiment:
    name: str
    dataset: str
    config: Path
    checkpoint: Optional[Path]
    manifest: Path
    view_manifest: Path
    image_size: int
    num_views: int = DEFAULT_NUM_VIEWS
    view_seed: int = DEFAULT_VIEW_SEED
    expected_scenes: Optional[int] = None
    paper_model: str = ""
    display_name: str = ""
    checkpoint_impl: str = ""
    overrides: List[str] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @property
    def scored_views(self) -> int:
        return self.num_views - 1          # view 0 only conditions


def load_registry(path) -> Dict[str, Experiment]:
    with open(path) as fh:
        doc = yaml.safe_load(fh) or {}
    defaults = doc.get("defaults", {}) or {}
    datasets = doc.get("datasets", {}) or {}
    ckpt_root = Path(os.path.expanduser(str(defaults.get("checkpoint_root", "."))))
    out: Dict[str, Experiment] = {}
    for entry in doc.get("experiments", []) or []:
        name = entry["name"]
        if name in out:
            raise ValueError(f"duplicate experiment {name!r} in {path}")
        ds_name = entry["dataset"]
        if ds_name not in datasets:
            raise ValueError(f"experiment {name!r} names unknown dataset {ds_name!r}")
        ds = datasets[ds_name]
        cfg = Path(entry["config"])
        if not cfg.is_absolute():
            cfg = REPO_ROOT / cfg
        ckpt = entry.get("checkpoint")
        ckpt_path = None
        if ckpt:
            ckpt_path = Path(ckpt)
            if not ckpt_path.is_absolute():
                ckpt_path = ckpt_root / ckpt_path
        out[name] = Experiment(
            name=name, dataset=ds_name, config=cfg, checkpoint=ckpt_path, manifest=Path(ds["manifest"]),
            view_manifest=Path(ds["view_manifest"]), image_size=int(ds.get("image_size", 256)),
            num_views=int(ds.get("num_views", defaults.get("num_views", DEFAULT_NUM_VIEWS))),
            view_seed=int(ds.get("view_seed", defaults.get("view_seed", DEFAULT_VIEW_SEED))),
            expected_scenes=ds.get("num_scenes"), paper_model=entry.get("paper_model", ""),
            display_name=entry.get("display_name", entry.get("paper_model", name)),
            checkpoint_impl=entry.get("checkpoint_impl", ""), overrides=list(entry.get("overrides", []) or []),
            raw=dict(entry))
    return out


def output_root(path, override=None) -> Path:
    if override is not None:
        return Path(override)
    with open(path) as fh:
        doc = yaml.safe_load(fh) or {}
    return Path((doc.get("defaults", {}) or {}).get("output_root", "eval_outputs"))


def preflight(exp: Experiment, require_checkpoint: bool = True) -> List[str]:
    """Everything a run needs must exist locally; a run never falls back to remote paths or other scenes."""
    problems = []
    if not exp.config.is_file():
        problems.append(f"config not found: {exp.config}")
    if require_checkpoint and (exp.checkpoint is None or not exp.checkpoint.is_file()):
        problems.append(f"checkpoint not found: {exp.checkpoint}")
    if not exp.manifest.is_file():
        problems.append(f"local manifest not found: {exp.manifest}")
    else:
        with open(exp.manifest) as fh:
            scenes = [ln.strip() for ln in fh if ln.strip()]
        remote = [s for s in scenes if "://" in s]
        if remote:
            problems.append(f"{len(remote)} manifest entries are remote paths (first: {remote[0]})")
        missing = [s for s in scenes if "://" not in s and not os.path.isfile(s)]
        if missing:
            problems.append(f"{len(missing)} scenes of the manifest are missing locally (first: {missing[0]})")
        if exp.expected_scenes is not None and len(scenes) != int(exp.expected_scenes):
            problems.append(f"manifest has {len(scenes)} scenes, the registry expects {exp.expected_scenes}")
    if not exp.view_manifest.is_file():
        problems.append(f"frozen view manifest not found: {exp.view_manifest}")
    return problems
