"""Named ranges for timelines: NVTX ranges (visible to Nsight tools) and ``torch.profiler`` record functions around
{chunk, layer read, chunk-boundary write, expert-parallel dispatch / combine, optimizer step}.

Off by default (a disabled range costs one attribute lookup); switch on with ``UTTT_B200_TRACE=1`` or
``trace.enable(True)``; the trainer's profiling flag enables it together with the torch profiler.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("UTTT_B200_TRACE", "0") == "1"


def enable(flag: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


def enabled() -> bool:
    return _ENABLED


@contextlib.contextmanager
def trace_range(name: str):
    if not _ENABLED:
        yield
        return
    use_nvtx = torch.cuda.is_available()
    if use_nvtx:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if use_nvtx:
            torch.cuda.nvtx.range_pop()
