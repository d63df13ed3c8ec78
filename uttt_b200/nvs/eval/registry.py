"""Experiment registry of the full-test evaluation (uttt_nvs/eval/common.py:58-170, experiments.yaml).

A registry is a YAML file in the reference's layout::

    version: 1
    defaults:
      checkpoint_root: /PATH/TO/CHECKPOINTS        # relative checkpoints are taken against it
      output_root: /PATH/TO/EVAL_OUTPUTS           # results go to <output_root>/<dataset>/<id>/
      seed: 9595                                   # bootstrap seed
      num_views: 24
    datasets:
      - id: gso
        local_manifest: /PATH/gso_local.txt
        view_manifest: /PATH/gso_views_seed9595_v24.json
        expected_scenes: 1019
        expected_rows: 23437                       # scenes x scored views
    experiments:
      - id: gso_uttt_moe_e32a2
        dataset: gso
        model: uttt_moe_e32a2
        paper_model: uTTT-MoE
        config: configs/nvs/width/obj/uttt_moe_e32a2.yaml      # relative to the repository root
        checkpoint: object/uttt_moe_e32a2/checkpoint.pt
        checkpoint_step: 24476
        checkpoint_impl: uttt_moe
        group: uttt_moe
        display_name: uTTT-MoE-e32a2
        expected_v_gap: null                       # optional; a non-null gap also needs allow_nonnull_v_gap: true

A registry written for the reference loads unchanged: its ``uttt_nvs/configs/...`` paths are looked up under
``configs/nvs/...`` when they do not exist as written.  The mapping form of ``datasets`` and the keys ``name``,
``manifest`` and ``num_scenes`` of earlier versions of this package are accepted too.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

import yaml

REPO_ROOT = Path(__file__).resolve().parents[3]
DEFAULT_REGISTRY = REPO_ROOT / "configs" / "nvs" / "eval" / "experiments.yaml"
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
    image_size: Optional[int] = None               # None: model.image_size of the config
    num_views: int = DEFAULT_NUM_VIEWS
    view_seed: int = DEFAULT_VIEW_SEED
    expected_scenes: Optional[int] = None
    expected_rows: Optional[int] = None
    paper_model: str = ""
    display_name: str = ""
    checkpoint_impl: str = ""
    overrides: List[str] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)
    dataset_raw: Dict[str, Any] = field(default_factory=dict)
    defaults: Dict[str, Any] = field(default_factory=dict)

    @property
    def id(self) -> str:
        return self.name

    @property
    def scored_views(self) -> int:
        return self.num_views - 1          # view 0 only conditions

    @property
    def model_name(self) -> str:
        return str(self.raw.get("paper_model", self.raw.get("model", self.name)))

    @property
    def bootstrap_seed(self) -> int:
        return int(self.defaults.get("seed", DEFAULT_VIEW_SEED))


def _resolve(path, base: Path) -> Path:
    p = Path(os.path.expanduser(str(path)))
    return p if p.is_absolute() else (base / p)


def _config_path(path) -> Path:
    p = _resolve(path, REPO_ROOT)
    if not p.exists():
        s = str(path).replace("\\", "/")
        if s.startswith("uttt_nvs/configs/"):
            alt = REPO_ROOT / "configs" / "nvs" / s[len("uttt_nvs/configs/"):]
            if alt.exists():
                return alt
    return p


def read_registry(path) -> Dict[str, Any]:
    """The YAML document with ``datasets`` normalised to a mapping by id; structural errors are raised here."""
    path = Path(os.path.expanduser(str(path)))
    with open(path, encoding="utf-8") as fh:
        doc = yaml.safe_load(fh)
    if not isinstance(doc, dict):
        raise ValueError(f"Registry must contain a mapping: {path}")
    for key in ("defaults", "datasets", "experiments"):
        if key not in doc:
            raise ValueError(f"Registry is missing top-level key {key!r}")
    doc["defaults"] = doc["defaults"] or {}
    if not isinstance(doc["experiments"], list):
        raise ValueError("registry.experiments must be a list")
    ds = doc["datasets"]
    if isinstance(ds, list):
        ids = [str(d["id"]) for d in ds]
        dup = sorted({i for i in ids if ids.count(i) > 1})
        if dup:
            raise ValueError(f"Duplicate dataset ids: {dup}")
        doc["datasets"] = {str(d["id"]): d for d in ds}
    elif isinstance(ds, dict):
        doc["datasets"] = {str(k): dict(v, id=str(k)) for k, v in ds.items()}
    else:
        raise ValueError("registry.datasets must be a mapping or list")
    ids = [str(e.get("id", e.get("name"))) for e in doc["experiments"]]
    dup = sorted({i for i in ids if ids.count(i) > 1})
    if dup:
        raise ValueError(f"Duplicate experiment ids: {dup}")
    return doc


def load_registry(path) -> Dict[str, Experiment]:
    doc = read_registry(path)
    defaults, datasets = doc["defaults"], doc["datasets"]
    ckpt_root = _resolve(defaults.get("checkpoint_root", "."), REPO_ROOT)
    out: Dict[str, Experiment] = {}
    for entry in doc["experiments"]:
        name = str(entry.get("id", entry.get("name")))
        ds_name = str(entry["dataset"])
        if ds_name not in datasets:
            raise KeyError(f"Unknown dataset {ds_name!r} in {name!r}")
        ds = datasets[ds_name]
        num_views = int(ds.get("num_views", defaults.get("num_views", DEFAULT_NUM_VIEWS)))
        scenes = ds.get("expected_scenes", ds.get("num_scenes"))
        rows = ds.get("expected_rows")
        if rows is None and scenes is not None:
            rows = int(scenes) * (num_views - 1)
        ckpt = entry.get("checkpoint")
        paper = str(entry.get("paper_model", entry.get("model", name)))
        out[name] = Experiment(
            name=name, dataset=ds_name, config=_config_path(entry["config"]),
            checkpoint=_resolve(ckpt, ckpt_root) if ckpt else None,
            manifest=_resolve(ds.get("local_manifest", ds.get("manifest")), REPO_ROOT),
            view_manifest=_resolve(ds["view_manifest"], REPO_ROOT),
            image_size=int(ds["image_size"]) if ds.get("image_size") else None, num_views=num_views,
            view_seed=int(ds.get("view_seed", defaults.get("view_seed", defaults.get("seed", DEFAULT_VIEW_SEED)))),
            expected_scenes=None if scenes is None else int(scenes), expected_rows=None if rows is None else int(rows),
            paper_model=paper, display_name=str(entry.get("display_name", paper)),
            checkpoint_impl=str(entry.get("checkpoint_impl", "") or ""), overrides=list(entry.get("overrides", []) or []),
            raw=dict(entry), dataset_raw=dict(ds), defaults=dict(defaults))
    return out


def resolve_experiment(path, experiment_id: str) -> Experiment:
    reg = load_registry(path)
    if experiment_id not in reg:
        raise KeyError(f"Expected one registry entry for {experiment_id!r}; known: {sorted(reg)[:8]} ...")
    return reg[experiment_id]


def select_experiments(path, datasets: Optional[Iterable[str]] = None) -> List[str]:
    allowed = set(datasets or [])
    return [e.name for e in load_registry(path).values() if not allowed or e.dataset in allowed]


def output_root(path, override=None) -> Path:
    if override is not None:
        return Path(os.path.expanduser(str(override)))
    return _resolve(read_registry(path)["defaults"].get("output_root", "eval_outputs"), REPO_ROOT)


def experiment_dir(root: Path, exp: Experiment) -> Path:
    """``<root>/<dataset>/<id>``; the shard i of a split run is evaluated with ``--output-root <shards>/shard_<i>``."""
    return Path(root) / exp.dataset / exp.name


def config_v_gap(cfg: Dict[str, Any]):
    return (((cfg.get("model") or {}).get("block_config") or {}).get("params") or {}).get("v_gap")


def validate_v_gap(exp: Experiment, cfg: Dict[str, Any]):
    """The attention gap of the model configuration must be the one the registry declares (``expected_v_gap``,
    default null), and a non-null gap needs ``allow_nonnull_v_gap: true`` on the entry."""
    actual = config_v_gap(cfg)
    expected = exp.raw.get("expected_v_gap", exp.raw.get("v_gap"))
    if actual != expected:
        raise ValueError(f"{exp.name}: expected v_gap={expected!r}, got {actual!r} from {exp.config}")
    if actual is not None and not bool(exp.raw.get("allow_nonnull_v_gap", False)):
        raise ValueError(f"{exp.name}: non-null v_gap={actual!r} requires an explicit allow_nonnull_v_gap "
                         f"registry declaration")
    return actual


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
        missing = [s for s in scenes if "://" not in s
                   and not os.path.isfile(s if os.path.isabs(s) else os.path.join(exp.manifest.parent, s))]
        if missing:
            problems.append(f"{len(missing)} scenes of the manifest are missing locally (first: {missing[0]})")
        if exp.expected_scenes is not None and len(scenes) != int(exp.expected_scenes):
            problems.append(f"manifest has {len(scenes)} scenes, the registry expects {exp.expected_scenes}")
    if not exp.view_manifest.is_file():
        problems.append(f"frozen view manifest not found: {exp.view_manifest}")
    return problems
