"""Static validation of every configuration file:  ``python -m uttt_b200.tools.check_configs [--catalog out.md]``.

Language-model JSON files are parsed into their config classes (which run the cross-field validation rules) and
checked for divisibility, expert bounds and a registered model type; job TOML files for the global-batch
arithmetic; view-synthesis YAML files for class-path resolution, divisibility, expert bounds and batch
arithmetic.  Needs no GPU and builds no model (the counterpart of tools/check_configs.py:63-152).
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from typing import List, Tuple

import yaml

try:
    import tomllib
except ModuleNotFoundError:  # pragma: no cover
    import tomli as tomllib

from ..config import load_config

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "configs")


def check_lm_json(path: str) -> List[str]:
    errs = []
    try:
        cfg = load_config(path)
    except Exception as exc:
        return [f"{path}: {exc}"]
    from ..models import registered_model_types
    if cfg.model_type not in registered_model_types():
        errs.append(f"{path}: model_type {cfg.model_type!r} has no registered model")
    if cfg.hidden_size % cfg.num_heads:
        errs.append(f"{path}: hidden_size not divisible by num_heads")
    if cfg.use_memory_block and cfg.hidden_size % cfg.fw_heads:
        errs.append(f"{path}: hidden_size not divisible by fw_num_heads")
    if cfg.max_position_embeddings % cfg.chunk_size and cfg.use_memory_block:
        errs.append(f"{path}: context length is not a whole number of chunks")
    e, k = getattr(cfg, "memory_num_experts", 1), getattr(cfg, "memory_num_active_experts", 1)
    if k > e:
        errs.append(f"{path}: more active experts than experts")
    if not errs:
        # a registration that resolves but a constructor that rejects the file only shows when the model is built
        import torch
        from ..models import build_model
        try:
            with torch.device("meta"):
                build_model(cfg)
        except Exception as exc:
            errs.append(f"{path}: the model cannot be built: {type(exc).__name__}: {exc}")
    return errs


def check_job_toml(path: str) -> List[str]:
    with open(path, "rb") as fh:
        job = tomllib.load(fh)
    tr = job.get("training", {})
    want = tr.get("expected_global_batch_size")
    if want is not None and want % (tr.get("batch_size", 1) * tr.get("gradient_accumulation_steps", 1)):
        return [f"{path}: expected_global_batch_size is not a multiple of batch_size x accumulation"]
    return []


def check_nvs_yaml(path: str) -> List[str]:
    from ..nvs.model import get_obj_by_name, resolve_model_class
    errs = []
    with open(path) as fh:
        cfg = yaml.safe_load(fh)
    m, tr = cfg["model"], cfg["training"]
    try:
        resolve_model_class(m.get("class_name"))
    except ValueError as exc:
        errs.append(f"{path}: {exc}")
    try:
        get_obj_by_name(m["block_config"]["type"])
    except Exception as exc:
        errs.append(f"{path}: cannot resolve {m['block_config']['type']}: {exc}")
    p = m["block_config"].get("params", {})
    size = m["image_size"] if isinstance(m["image_size"], int) else m["image_size"][0]
    if size % m["patch_size"]:
        errs.append(f"{path}: image_size not divisible by patch_size")
    if m["dim"] % p.get("attn_head_dim", m["dim"]):
        errs.append(f"{path}: dim not divisible by attn_head_dim")
    if m["dim"] % (p.get("fw_head_dim") or m["dim"]):
        errs.append(f"{path}: dim not divisible by fw_head_dim")
    if p.get("num_active_experts", 1) > p.get("num_experts", 1):
        errs.append(f"{path}: more active experts than experts")
    if not isinstance(cfg.get("exp_name"), str) or not cfg["exp_name"]:
        errs.append(f"{path}: exp_name must be a non-empty string")
    counts_ok = True
    for key in ("total_batch_size", "batch_size_per_gpu", "grad_accum_steps", "num_views", "eval_num_views",
                "max_fwdbwd_passes", "checkpoint_every"):
        if key in tr and (type(tr[key]) is not int or tr[key] < 1):
            errs.append(f"{path}: training.{key} must be a positive integer, got {tr[key]!r}")
            counts_ok = False
    if counts_ok and tr["total_batch_size"] % (tr["batch_size_per_gpu"] * tr.get("grad_accum_steps", 1)):
        errs.append(f"{path}: total_batch_size is not reachable with batch_size_per_gpu x grad_accum_steps")
    if type(p.get("num_experts", 1)) is not int or p.get("num_experts", 1) < 1:
        errs.append(f"{path}: num_experts must be a positive integer")
    if p.get("aggregate_write") and p.get("pool_mode", "shared") != "shared":
        errs.append(f"{path}: aggregate_write requires a shared pool")
    if not errs:
        # the stack's constructor is the authority on its parameters: build it without allocating anything
        import copy
        import torch
        from ..nvs.model import LVSMModel
        probe = copy.deepcopy(cfg)
        probe["training"].update(perceptual_loss_weight=0.0, lpips_loss_weight=0.0)   # their networks need weight files
        try:
            with torch.device("meta"):
                LVSMModel(probe)
        except Exception as exc:
            errs.append(f"{path}: the model cannot be built: {type(exc).__name__}: {exc}")
    return errs


def check_all(root: str = ROOT) -> Tuple[int, List[str]]:
    errs: List[str] = []
    n = 0
    for path in sorted(glob.glob(os.path.join(root, "lm", "**", "*.json"), recursive=True)):
        errs += check_lm_json(path)
        n += 1
    for path in sorted(glob.glob(os.path.join(root, "lm", "**", "*.toml"), recursive=True)):
        errs += check_job_toml(path)
        n += 1
    for path in sorted(glob.glob(os.path.join(root, "nvs", "**", "*.yaml"), recursive=True)):
        if os.path.basename(path).startswith(("datasets.", "api_keys.")):   # registries / keys, not run configurations
            continue
        if os.sep + "eval" + os.sep in path:
            errs += check_eval_registry(path)
        else:
            errs += check_nvs_yaml(path)
        n += 1
    return n, errs


def check_eval_registry(path: str) -> List[str]:
    """Every entry of an evaluation registry names a known dataset and a configuration file that exists."""
    from ..nvs.eval.registry import load_registry
    try:
        reg = load_registry(path)
    except Exception as exc:
        return [f"{path}: {exc}"]
    return [f"{path}: {e.name}: config {e.config} not found" for e in reg.values() if not e.config.is_file()]


def catalog(root: str = ROOT) -> str:
    lines = ["# Configuration catalog", "", "| file | kind | summary |", "|---|---|---|"]
    for path in sorted(glob.glob(os.path.join(root, "**", "*.*"), recursive=True)):
        rel = os.path.relpath(path, root)
        if path.endswith(".json"):
            c = load_config(path)
            extra = f", E={c.memory_num_experts} top-{c.memory_num_active_experts}" if hasattr(c, "memory_num_experts") else ""
            lines.append(f"| {rel} | lm:{c.model_type} | d={c.hidden_size} L={c.num_hidden_layers} chunk={c.chunk_size}{extra} |")
        elif os.path.basename(path).startswith("datasets."):
            lines.append(f"| {rel} | registry | dataset paths, to be copied to datasets.yaml and filled in |")
        elif os.path.basename(path).startswith("api_keys."):
            lines.append(f"| {rel} | keys | logging key, to be copied to api_keys.yaml and filled in |")
        elif path.endswith(".yaml") and os.sep + "eval" + os.sep in path:
            with open(path) as fh:
                c = yaml.safe_load(fh)
            lines.append(f"| {rel} | nvs-eval | registry of {len(c.get('experiments', []))} evaluations |")
        elif path.endswith(".yaml"):
            with open(path) as fh:
                c = yaml.safe_load(fh)
            lines.append(f"| {rel} | nvs | {c['model']['block_config']['type'].rsplit('.', 2)[-2]} dim={c['model']['dim']} "
                         f"L={c['model']['layers']} {c['model']['image_size']}px |")
        elif path.endswith(".toml"):
            lines.append(f"| {rel} | job | |")
    return "\n".join(lines) + "\n"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--root", default=ROOT)
    ap.add_argument("--catalog", default=None)
    ap.add_argument("--check-catalog", action="store_true")
    args = ap.parse_args()
    n, errs = check_all(args.root)
    for e in errs:
        print("ERROR", e)
    print(f"checked {n} configuration files: {len(errs)} problem(s)")
    cat_path = args.catalog or os.path.join(args.root, "CATALOG.md")
    if args.check_catalog:
        if not os.path.exists(cat_path) or open(cat_path).read() != catalog(args.root):
            print("ERROR configuration catalog is stale; regenerate with --catalog")
            return 1
    elif args.catalog:
        with open(cat_path, "w") as fh:
            fh.write(catalog(args.root))
    return 1 if errs else 0


if __name__ == "__main__":
    sys.exit(main())
