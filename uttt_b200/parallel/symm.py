"""Symmetric (peer-mapped) memory heap and the fused gradient / parameter collectives on it.

One contiguous buffer per rank is allocated with ``torch.distributed._symmetric_memory`` and
exchanged once; every rank then holds the base address of every peer's buffer, and sub-buffers
(flat parameter and gradient buffers, expert-parallel staging) are bump-allocated at identical
offsets on all ranks.  Kernels receive the list of peer addresses and use plain loads/stores over
NVLink; cross-rank ordering comes from tiny stream-ordered NCCL all-reduces, so no kernel of this
module ever spins on a peer.

Where the allocation is also bound to an NVLink multicast object (``multicast_ptr`` of the rendezvous
handle, present when the fabric supports NVLS) the two optimizer-step kernels can use ``multimem``
instructions instead: the gradient sum is formed inside the switch and the updated parameters are
written to all ranks with one store.  This form is opt-in (``UTTT_B200_MULTIMEM=1`` or
``SymmetricHeap(use_multimem=True)``) because a bf16 gradient sum comes back rounded to bf16 (fp32
accumulation inside the switch), where the peer-pointer form keeps the fp32 sum.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops._ext import load


class SymmetricHeap:
    def __init__(self, device: torch.device, group=None, capacity_bytes: int = 0,
                 use_multimem: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem
        if capacity_bytes <= 0:
            raise ValueError("SymmetricHeap needs its capacity up front")
        self.device = device
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.capacity = (capacity_bytes + 4095) // 4096 * 4096
        self.buffer = symm_mem.empty(self.capacity, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.base_ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if use_multimem is None:
            use_multimem = os.environ.get("UTTT_B200_MULTIMEM", "0") == "1"
        # every rank must take the same form: the switch reduces over all bound ranks
        self.use_multimem = bool(use_multimem) and self.multicast_ptr != 0
        self.cursor = 0
        self._token = torch.zeros(1, device=device, dtype=torch.float32)
        self.ext = load(required=True)

    # ------------------------------------------------------------------ allocation
    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        item = torch.empty((), dtype=dtype).element_size()
        start = (self.cursor + 1023) // 1024 * 1024
        nbytes = numel * item
        if start + nbytes > self.capacity:
            raise MemoryError("symmetric heap exhausted")
        self.cursor = start + nbytes
        t = self.buffer[start:start + nbytes].view(dtype)
        t._symm_offset = start          # byte offset, identical on every rank
        return t

    def peer_ptrs(self, t: torch.Tensor) -> List[int]:
        off = t.data_ptr() - self.buffer.data_ptr()
        return [b + off for b in self.base_ptrs]

    def multicast_addr(self, t: torch.Tensor) -> int:
        """Address of ``t`` in the multicast mapping (0 when the multimem form is off)."""
        if not self.use_multimem:
            return 0
        return self.multicast_ptr + (t.data_ptr() - self.buffer.data_ptr())

    def finalize(self) -> None:
        self.barrier()

    def barrier(self) -> None:
        """Stream-ordered barrier over the group (a scalar all-reduce): every rank's earlier work on the
        current stream is complete on all ranks before any later work starts."""
        dist.all_reduce(self._token, group=self.group)

    # ------------------------------------------------------------------ fused collectives
    def reduce_scatter_sumsq(self, unit, src: torch.Tensor, scale: float, sumsq: torch.Tensor) -> torch.Tensor:
        """This rank's shard of sum_r grad_r * scale (fp32), adding its squared norm into ``sumsq``."""
        out = torch.empty(unit.shard_numel, dtype=torch.float32, device=self.device)
        lo, _ = unit.shard_range
        buf = unit.grad if src.data_ptr() == unit.grad.data_ptr() else unit.grad_accum
        self.ext.rs_sumsq(self.peer_ptrs(buf), self.rank, lo, out, float(scale), sumsq, src.dtype == torch.bfloat16,
                          self.multicast_addr(buf))
        return out

    def adamw_scatter(self, unit, g: torch.Tensor, lr: float, opt, step: int, gscale: torch.Tensor,
                      apply: torch.Tensor, decay_hi: int) -> None:
        lo, _ = unit.shard_range
        self.ext.adamw_scatter(unit.master, g, unit.exp_avg, unit.exp_avg_sq, self.peer_ptrs(unit.compute),
                               self.rank, lo, unit.compute.dtype == torch.bfloat16, float(lr), opt.beta1, opt.beta2,
                               opt.eps, opt.weight_decay, int(step), gscale, apply, int(decay_hi),
                               self.multicast_addr(unit.compute))
