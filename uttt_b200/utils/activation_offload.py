"""Activation offloading to pinned host memory (uttt_llm/flame/models/activation_offloading.py:30-447; in the
reference only the ``--activation_offload.mode`` flag exists, no call site uses it).

``with offload_activations(min_bytes=...):`` wraps a forward pass: tensors that autograd saves for backward and that
are at least ``min_bytes`` large are copied to pinned host memory on a side stream and brought back (on the same
side stream, ordered before their use) when backward needs them.  Parameters and small tensors stay on the
device.  On CPU tensors it is a no-op.  With the 180 GB of a B200 the 760M / 32K benchmark does not need it; it
serves larger per-GPU batches.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch


class _Offloader:
    def __init__(self, min_bytes: int, stream: Optional["torch.cuda.Stream"], fp32_only: bool = False):
        self.fp32_only = fp32_only
        self.min_bytes = int(min_bytes)
        self.stream = stream
        self.bytes_offloaded = 0
        self.tensors_offloaded = 0

    def pack(self, t: torch.Tensor):
        if (not t.is_cuda) or isinstance(t, torch.nn.Parameter) or t.numel() * t.element_size() < self.min_bytes:
            return t
        if self.fp32_only and (t.dtype != torch.float32 or not t.is_contiguous()):
            return t            # master states only; broadcast views would be materialised at full size
        stream = self.stream or torch.cuda.Stream(t.device)
        self.stream = stream
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        stream.wait_stream(torch.cuda.current_stream(t.device))
        with torch.cuda.stream(stream):
            host.copy_(t, non_blocking=True)
            done = torch.cuda.Event()
            done.record(stream)
        t.record_stream(stream)                       # the device copy may be freed once the transfer has read it
        self.bytes_offloaded += t.numel() * t.element_size()
        self.tensors_offloaded += 1
        return (host, t.device, done)

    def unpack(self, packed):
        if isinstance(packed, torch.Tensor):
            return packed
        host, device, done = packed
        stream = self.stream
        with torch.cuda.stream(stream):
            stream.wait_event(done)
            out = host.to(device, non_blocking=True)
        torch.cuda.current_stream(device).wait_stream(stream)
        out.record_stream(torch.cuda.current_stream(device))
        return out


@contextlib.contextmanager
def offload_activations(min_bytes: int = 1 << 20, stream: Optional["torch.cuda.Stream"] = None, enabled: bool = True,
                        fp32_only: bool = False):
    """Context manager; yields the offloader (``bytes_offloaded`` / ``tensors_offloaded`` counters).
    ``fp32_only`` restricts it to contiguous fp32 tensors (the fast-weight master copies)."""
    off = _Offloader(min_bytes, stream, fp32_only)
    if not enabled:
        yield off
        return
    with torch.autograd.graph.saved_tensors_hooks(off.pack, off.unpack):
        yield off
