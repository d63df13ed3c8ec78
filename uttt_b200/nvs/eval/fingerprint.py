"""Runtime fingerprint stored beside every evaluation (uttt_nvs/eval/runtime_fingerprint.py, common.py:245-275):
enough to tell two runs apart that should have been identical.

* :func:`deterministic_runtime_fingerprint`: only properties that decide the numbers (interpreter and library
  versions, CUDA / cuDNN builds, GPU model and compute capability, driver, numeric flags, whether the native
  kernels are loaded).  Nothing that names a machine, a process or a shard is in it, so all shards of a run and
  reruns elsewhere on equal software hash the same; :func:`validate_runtime_fingerprint` rejects such keys.
* :func:`runtime_fingerprint`: the wider record for people (command line, git state, environment).
* digests: :func:`file_sha256`, :func:`canonical_json_sha256`, :func:`evaluation_code_sha256` (the evaluator's own
  sources, uncommitted edits included).
"""
from __future__ import annotations

import hashlib
import json
import os
import platform
import subprocess
import sys
from pathlib import Path
from typing import Any, Dict, Mapping

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


RUNTIME_SCHEMA = "uttt-b200-runtime-fingerprint-v1"
_FORBIDDEN = ("hostname", "uuid", "pci", "bus", "ordinal", "process", "shard")
_FLAGS = ("deterministic_algorithms", "cudnn_deterministic", "cudnn_benchmark", "cuda_matmul_allow_tf32",
          "cudnn_allow_tf32", "default_dtype")
_RUNTIME_KEYS = ("schema_version", "python", "python_implementation", "torch", "torchvision", "numpy", "pillow",
                 "torch_cuda_build", "cudnn", "gpu_model", "gpu_compute_capability", "nvidia_driver", "native_kernels",
                 "numeric_flags")


def canonical_json_sha256(value: Any) -> str:
    return hashlib.sha256(json.dumps(value, ensure_ascii=False, sort_keys=True,
                                     separators=(",", ":")).encode("utf-8")).hexdigest()


def git_commit(repo_root=None) -> str:
    root = Path(repo_root) if repo_root else Path(__file__).resolve().parents[3]
    return _git(root, "rev-parse", "HEAD") or "unknown"


def evaluation_code_sha256() -> str:
    """Digest over the sources of this package (relative name, NUL, bytes, NUL per file, sorted by name)."""
    here = Path(__file__).resolve().parent
    h = hashlib.sha256()
    for path in sorted(here.glob("*.py")):
        h.update(f"nvs/eval/{path.name}".encode())
        h.update(b"\0")
        h.update(path.read_bytes())
        h.update(b"\0")
    return h.hexdigest()


def _version(*names: str) -> str:
    import importlib.metadata as md
    for n in names:
        try:
            return md.version(n)
        except md.PackageNotFoundError:
            continue
    return "not-installed"


def _driver_version() -> str:
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader,nounits"],
                             check=True, capture_output=True, text=True, timeout=10).stdout
    except (FileNotFoundError, subprocess.SubprocessError):
        return "unavailable"
    found = sorted({ln.strip() for ln in out.splitlines() if ln.strip()})
    return ",".join(found) if found else "unavailable"


def deterministic_runtime_fingerprint(device="cpu") -> Dict[str, Any]:
    import numpy as np
    dev = torch.device(device)
    gpu, cap = None, None
    if dev.type == "cuda":
        if not torch.cuda.is_available():
            raise RuntimeError("CUDA runtime fingerprint requested without CUDA")
        idx = torch.cuda.current_device() if dev.index is None else dev.index
        gpu, cap = torch.cuda.get_device_name(idx), list(torch.cuda.get_device_capability(idx))
    from ...ops._ext import available
    cudnn = torch.backends.cudnn.version() if torch.backends.cudnn.is_available() else None
    return {
        "schema_version": RUNTIME_SCHEMA, "python": platform.python_version(),
        "python_implementation": platform.python_implementation(), "torch": str(torch.__version__),
        "torchvision": _version("torchvision"), "numpy": str(np.__version__), "pillow": _version("pillow", "Pillow"),
        "torch_cuda_build": str(torch.version.cuda), "cudnn": None if cudnn is None else int(cudnn),
        "gpu_model": gpu, "gpu_compute_capability": cap, "nvidia_driver": _driver_version(),
        "native_kernels": bool(available()),
        "numeric_flags": {
            "deterministic_algorithms": bool(torch.are_deterministic_algorithms_enabled()),
            "cudnn_deterministic": bool(torch.backends.cudnn.deterministic),
            "cudnn_benchmark": bool(torch.backends.cudnn.benchmark),
            "cuda_matmul_allow_tf32": bool(torch.backends.cuda.matmul.allow_tf32),
            "cudnn_allow_tf32": bool(torch.backends.cudnn.allow_tf32),
            "default_dtype": str(torch.get_default_dtype())}}


def runtime_fingerprint_sha256(payload: Mapping[str, Any]) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"),
                                     ensure_ascii=True).encode("utf-8")).hexdigest()


def validate_runtime_fingerprint(payload: Mapping[str, Any], require_cuda: bool = True) -> None:
    """Exact key set, typed values, and no key anywhere that could carry host / process / shard identity."""
    if not isinstance(payload, Mapping):
        raise ValueError("runtime fingerprint must be an object")

    def walk(v):
        if isinstance(v, Mapping):
            for k, inner in v.items():
                if any(tok in str(k).lower() for tok in _FORBIDDEN):
                    raise ValueError(f"forbidden runtime fingerprint key: {k}")
                walk(inner)
        elif isinstance(v, (list, tuple)):
            for inner in v:
                walk(inner)

    walk(payload)
    if set(payload) != set(_RUNTIME_KEYS):
        raise ValueError(f"runtime fingerprint fields changed; missing={sorted(set(_RUNTIME_KEYS) - set(payload))}, "
                         f"extra={sorted(set(payload) - set(_RUNTIME_KEYS))}")
    if payload["schema_version"] != RUNTIME_SCHEMA:
        raise ValueError("runtime fingerprint schema version changed")
    for k in ("python", "python_implementation", "torch", "torchvision", "numpy", "pillow", "torch_cuda_build",
              "nvidia_driver"):
        if not isinstance(payload[k], str) or not payload[k]:
            raise ValueError(f"runtime fingerprint {k} must be a nonempty string")
    flags = payload["numeric_flags"]
    if not isinstance(flags, Mapping) or set(flags) != set(_FLAGS):
        raise ValueError("runtime numeric flag schema changed")
    for k in _FLAGS[:-1]:
        if not isinstance(flags[k], bool):
            raise ValueError(f"runtime numeric flag {k} must be boolean")
    if not isinstance(flags["default_dtype"], str) or not flags["default_dtype"]:
        raise ValueError("runtime default_dtype must be a nonempty string")
    if not isinstance(payload["native_kernels"], bool):
        raise ValueError("runtime native_kernels must be boolean")
    cudnn, cap = payload["cudnn"], payload["gpu_compute_capability"]
    if cudnn is not None and (not isinstance(cudnn, int) or isinstance(cudnn, bool)):
        raise ValueError("runtime cuDNN version must be integer or null")
    if require_cuda:
        if not isinstance(payload["gpu_model"], str) or not payload["gpu_model"]:
            raise ValueError("formal CUDA runtime lacks GPU model")
        if not isinstance(cap, list) or len(cap) != 2 or any(not isinstance(v, int) for v in cap):
            raise ValueError("formal CUDA runtime lacks compute capability")
        if payload["torch_cuda_build"] in ("None", "none", ""):
            raise ValueError("formal CUDA runtime lacks torch CUDA build")
        if cudnn is None:
            raise ValueError("formal CUDA runtime lacks cuDNN")
        if payload["nvidia_driver"] == "unavailable":
            raise ValueError("formal CUDA runtime lacks NVIDIA driver")
    elif payload["gpu_model"] is not None and not isinstance(payload["gpu_model"], str):
        raise ValueError("GPU model must be a string or null")


NATURAL_OUTPUT_IDENTITY_ASSET_KEYS = ("registry_sha256", "checkpoint_sha256", "config_sha256", "dataset_manifest_sha256",
                                      "view_manifest_sha256", "code_commit", "redundancy_code_sha256")


def natural_output_source_fingerprint_sha256(*, experiment_id: str, protocol_version: str, run_signature: str,
                                             identity_assets: Mapping[str, Any], runtime_sha256: str,
                                             scene_count: int, scene_file_sha256: Mapping[str, str]) -> str:
    """Path-independent identity of a folder of per-scene model outputs (uttt_nvs/eval/common.py:277-360): which
    experiment under which protocol and run signature produced it, from which assets (exactly the seven keys of
    ``NATURAL_OUTPUT_IDENTITY_ASSET_KEYS``), on which runtime, and the digest of every scene file by base name.
    Any malformed part is an error, so two folders hash alike only when all of it agrees."""
    scalars = {"experiment_id": experiment_id, "protocol_version": protocol_version, "run_signature": run_signature,
               "runtime_sha256": runtime_sha256}
    bad = [k for k, v in scalars.items() if not isinstance(v, str) or not v]
    if bad:
        raise ValueError(f"natural-output fingerprint has invalid fields {bad}")
    if not isinstance(identity_assets, Mapping):
        raise ValueError("natural-output identity_assets must be an object")
    if set(identity_assets) != set(NATURAL_OUTPUT_IDENTITY_ASSET_KEYS):
        raise ValueError(f"natural-output identity_assets must contain exactly {sorted(NATURAL_OUTPUT_IDENTITY_ASSET_KEYS)}")
    if any(not isinstance(identity_assets[k], str) or not identity_assets[k] for k in NATURAL_OUTPUT_IDENTITY_ASSET_KEYS):
        raise ValueError("natural-output identity asset values must be non-empty strings")
    if isinstance(scene_count, bool) or not isinstance(scene_count, int) or scene_count <= 0:
        raise ValueError("natural-output scene_count must be a positive integer")
    if not isinstance(scene_file_sha256, Mapping) or len(scene_file_sha256) != scene_count:
        raise ValueError("natural-output scene_file_sha256 must contain exactly scene_count entries")
    for name, digest in scene_file_sha256.items():
        if not isinstance(name, str) or not name or os.path.basename(name) != name or not isinstance(digest, str) \
                or not digest:
            raise ValueError("natural-output scene hashes require basename keys and non-empty strings")
    return canonical_json_sha256({**scalars,
                                  "identity_assets": {k: identity_assets[k] for k in NATURAL_OUTPUT_IDENTITY_ASSET_KEYS},
                                  "scene_count": scene_count, "scene_file_sha256": dict(scene_file_sha256)})
