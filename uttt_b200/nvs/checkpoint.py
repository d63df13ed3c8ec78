"""Checkpoints of the view-synthesis trainer: ``<out_dir>/ckpt_<step:016d>.pt`` holding
``{model, optimizer, lr_scheduler, fwdbwd_pass_step, param_update_step}``; atomic publish, numeric
discovery, count-based retention, newest-readable fallback, reset modes
(uttt_nvs/train/checkpoint.py:14-254)."""
from __future__ import annotations

import os
import re
import tempfile
from typing import List, Tuple

import torch

_PREFIXES = ("_checkpoint_wrapped_module.", "_orig_mod.")


def clean_key(key: str) -> str:
    for p in _PREFIXES:
        key = key.replace(p, "")
    while key.startswith("module."):
        key = key[len("module."):]
    return key


def checkpoint_job(out_dir, model, optimizer, lr_scheduler, fwdbwd_pass_step: int, param_update_step: int) -> str:
    model = getattr(model, "module", model)
    state = {clean_key(k): v for k, v in model.state_dict().items()}
    blob = {"model": state, "optimizer": optimizer.state_dict(), "lr_scheduler": lr_scheduler.state_dict(),
            "fwdbwd_pass_step": fwdbwd_pass_step, "param_update_step": param_update_step}
    os.makedirs(out_dir, exist_ok=True)
    final = os.path.join(out_dir, f"ckpt_{fwdbwd_pass_step:016}.pt")
    tmp = None
    try:
        with tempfile.NamedTemporaryFile(dir=out_dir, prefix=".ckpt_", suffix=".tmp", delete=False) as fh:
            tmp = fh.name
            torch.save(blob, fh)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, final)
    finally:
        if tmp is not None and os.path.exists(tmp):
            os.remove(tmp)
    return final


def find_checkpoints(out_dir) -> List[str]:
    if not os.path.isdir(out_dir):
        return []
    found = []
    for name in os.listdir(out_dir):
        m = re.fullmatch(r"ckpt_(\d+)\.pt", name)
        path = os.path.join(out_dir, name)
        if m and os.path.isfile(path):
            found.append((int(m.group(1)), path))
    return [p for _, p in sorted(found)]


def select_resume_path(out_dir, load_path: str = "", config_load_path: str = "") -> str:
    """An existing run wins over an explicit checkpoint, which wins over ``training.load``."""
    if find_checkpoints(out_dir):
        return out_dir
    return load_path or config_load_path or ""


def delete_previous_job(out_dir, fwdbwd_pass_step: int, save_last_n_ckpts: int = 1) -> None:
    if type(save_last_n_ckpts) is not int or save_last_n_ckpts < 1:
        raise ValueError("save_last_n_ckpts must be a positive integer")
    if not os.path.exists(out_dir):
        return
    keep = [p for p in find_checkpoints(out_dir) if int(os.path.basename(p)[5:-3]) <= fwdbwd_pass_step]
    for p in keep[:-save_last_n_ckpts]:
        os.remove(p)


def resume_job(load_path, model, optimizer, lr_scheduler, reset_training_state: bool = False,
               load_optimizer_state_when_reset_training_state: bool = False) -> Tuple[object, object, int, int]:
    """Returns (optimizer, lr_scheduler, fwdbwd_pass_step, param_update_step).  Empty path = from scratch; a
    directory is searched newest-first and falls back to older files when one cannot be read; nothing
    readable raises."""
    if not load_path:
        return optimizer, lr_scheduler, 0, 0
    load_path = os.fspath(load_path)
    if os.path.isdir(load_path):
        paths = find_checkpoints(load_path)
        if not paths:
            raise FileNotFoundError(f"No ckpt_<step>.pt checkpoints in {load_path}")
    else:
        if not load_path.endswith(".pt"):
            raise ValueError(f"Checkpoint path must be a .pt file or directory: {load_path}")
        if not os.path.isfile(load_path):
            raise FileNotFoundError(f"Checkpoint does not exist: {load_path}")
        paths = [load_path]
    blob, last = None, None
    for path in reversed(paths):
        try:
            blob = torch.load(path, map_location="cpu", weights_only=False)
            break
        except Exception as exc:                      # a truncated newest file: fall back to the one before it
            last = exc
            print(f"Failed to load {path} ({type(exc).__name__}); trying the next checkpoint in reverse order",
                  flush=True)
    if blob is None:
        raise RuntimeError(f"Failed to load any checkpoint in {load_path}; all ckpt paths: {paths}") from last
    target = getattr(model, "module", model)
    state = {clean_key(k): v for k, v in blob["model"].items()}
    target.load_state_dict(state, strict=False)

    def load_optimizer() -> bool:
        """A state that does not fit (another architecture, another layout) is skipped with a warning, as in
        the reference: training continues with fresh moments."""
        try:
            try:
                optimizer.load_state_dict(blob["optimizer"], model_state=state)
            except TypeError:
                optimizer.load_state_dict(blob["optimizer"])
            return True
        except (ValueError, KeyError) as exc:
            print(f"[WARNING] Failed to load optimizer state dict (likely a parameter mismatch): {exc}\n"
                  f"Skipping optimizer state restore.", flush=True)
            return False

    if reset_training_state:
        if load_optimizer_state_when_reset_training_state:
            load_optimizer()
        return optimizer, lr_scheduler, 0, 0
    load_optimizer()
    lr_scheduler.load_state_dict(blob["lr_scheduler"])
    return optimizer, lr_scheduler, int(blob["fwdbwd_pass_step"]), int(blob["param_update_step"])
