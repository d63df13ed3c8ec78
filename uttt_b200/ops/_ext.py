"""Loader for the in-tree sm_100a extension (``uttt_b200/ops/_C*.so``).

The extension is built by ``python -m uttt_b200.ops.build`` (or ``__graft_entry__.build()``)
into the package directory so that it travels with the source tree.  On a machine with a
CUDA device the ops refuse to run without it; on CPU-only machines the torch statements in
:mod:`uttt_b200.ops.reference` are the implementation.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import threading

import torch

_LOCK = threading.Lock()
_MOD = None
_ERR: Exception | None = None
_TRIED = False


def _find_so() -> str | None:
    here = os.path.dirname(os.path.abspath(__file__))
    cands = sorted(glob.glob(os.path.join(here, "_C*.so")))
    return cands[-1] if cands else None


def load(required: bool = False):
    """Return the extension module, or ``None`` when it is not built / not loadable."""
    global _MOD, _ERR, _TRIED
    with _LOCK:
        if not _TRIED:
            _TRIED = True
            path = _find_so()
            if path is None:
                _ERR = FileNotFoundError("uttt_b200/ops/_C*.so not found; run `python -m uttt_b200.ops.build`")
            else:
                try:
                    spec = importlib.util.spec_from_file_location("uttt_b200.ops._C", path)
                    mod = importlib.util.module_from_spec(spec)
                    spec.loader.exec_module(mod)
                    _MOD = mod
                except Exception as exc:  # pragma: no cover - depends on the box
                    _ERR = exc
    if _MOD is None and required:
        raise RuntimeError(f"the uttt_b200 CUDA extension is required on a GPU machine but is unavailable: {_ERR}")
    return _MOD


def available() -> bool:
    return load() is not None


def cuda_ext(*tensors: torch.Tensor):
    """Extension module if the call should run on the GPU kernels, else ``None`` (CPU tensors).

    Raises when a CUDA tensor is given but the extension cannot be loaded, unless
    ``UTTT_B200_ALLOW_TORCH_FALLBACK=1`` is set (debug only).
    """
    if not any(t is not None and t.is_cuda for t in tensors):
        return None
    mod = load()
    if mod is None:
        if os.environ.get("UTTT_B200_ALLOW_TORCH_FALLBACK") == "1":
            return None
        load(required=True)
    return mod


def has(name: str) -> bool:
    mod = load()
    return mod is not None and hasattr(mod, name)
