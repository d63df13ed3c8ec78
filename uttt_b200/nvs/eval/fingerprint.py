"""Runtime fingerprint stored beside every evaluation (uttt_nvs/eval/runtime_fingerprint.py): enough to tell
two runs apart that should have been identical."""
from __future__ import annotations

import hashlib
import json
import os
import platform
import subprocess
import sys
from pathlib import Path
from typing import Any, Dict

import torch


def _git(root: Path, *args: str) -> str:
    try:
        return subprocess.run(["git", "-C", str(root), *args], capture_output=True, text=True, timeout=10).stdout.strip()
    except Exception:
        return ""


def file_sha256(path, limit_bytes: int = 0) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        remaining = limit_bytes or None
        while True:
            chunk = fh.read(1 << 20 if remaining is None else min(1 << 20, remaining))
            if not chunk:
                break
            h.update(chunk)
            if remaining is not None:
                remaining -= len(chunk)
                if remaining <= 0:
                    break
    return h.hexdigest()


def runtime_fingerprint(repo_root=None, device: str = "cpu") -> Dict[str, Any]:
    root = Path(repo_root) if repo_root else Path(__file__).resolve().parents[3]
    fp: Dict[str, Any] = {
        "python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
        "cuda": torch.version.cuda, "cudnn": torch.backends.cudnn.version() if torch.backends.cudnn.is_available() else None,
        "git_commit": _git(root, "rev-parse", "HEAD"), "git_dirty": bool(_git(root, "status", "--porcelain")),
        "argv": list(sys.argv), "env": {k: os.environ[k] for k in ("CUDA_VISIBLE_DEVICES", "NCCL_NVLS_ENABLE")
                                        if k in os.environ},
        "tf32_matmul": torch.backends.cuda.matmul.allow_tf32, "deterministic": torch.are_deterministic_algorithms_enabled(),
    }
    if device.startswith("cuda") and torch.cuda.is_available():
        idx = torch.device(device).index or 0
        props = torch.cuda.get_device_properties(idx)
        fp["gpu"] = {"name": props.name, "capability": f"{props.major}.{props.minor}",
                     "memory_gib": round(props.total_memory / 2 ** 30, 1), "sms": props.multi_processor_count}
    from ...ops._ext import available
    fp["native_kernels"] = bool(available())
    return fp


def write_fingerprint(path, **kwargs) -> Dict[str, Any]:
    fp = runtime_fingerprint(**kwargs)
    with open(path, "w") as fh:
        json.dump(fp, fh, indent=1, sort_keys=True)
    return fp
