"""Expert parallelism for the routed fast-weight pool.

The reference keeps the whole pool state of a sequence on the data-parallel rank that owns the sequence (it has
no expert parallelism).  Here the experts can be sharded over the ``P`` ranks of an expert-parallel group: rank
``p`` owns experts ``[p * E/P, (p + 1) * E/P)`` of every sequence of the group, so a rank holds the state of
``P * B`` sequences x ``E / P`` experts, the grouped GEMMs and the Newton-Schulz updates of an expert run on its
owner, and routed rows travel to the owner and back.

Owner-side layout: groups ``g' = (source rank, sequence, local expert)``, each padded to a multiple of 128 rows,
dense and in that order; it is described by an ordinary ``GroupPlan`` so that the grouped GEMM kernels are used
unchanged with the state reshaped to ``[P * B * E/P, ...]``.

Two transports with identical semantics:

* ``peer``  - the kernels of ``ops/csrc/ep.cu`` over a symmetric heap: *dispatch* permutes and sends in one pass
  (each routed copy is stored over NVLink at its final position in the owner's buffer), *combine* receives,
  un-permutes and applies the gate-weighted sum in one pass (loads from the owners' buffers).  Ranks are ordered
  by tiny stream-ordered collectives around the kernels; no kernel waits on a peer.
* ``a2a``   - local permute + ``all_to_all_single`` + local un-permute, built from differentiable torch ops
  (works on ``gloo``; the baseline the fused kernels are compared against).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import functional as F_ops
from ..ops import reference as ref
from ..ops._ext import load
from ..utils.trace import trace_range

TILE = ref.TILE_ROWS


@dataclass
class EPPlan:
    local: F_ops.GroupPlan          # sender-side plan over groups b * E + e
    owner: F_ops.GroupPlan          # owner-side plan over groups (s * B + b) * El + el
    idx: torch.Tensor               # [R, k] int32 expert of every routed copy
    sizes32: torch.Tensor           # [B * E] int32 sizes of the sender's groups
    rows_per_batch: int
    remote_start: Optional[torch.Tensor] = None     # peer transport: [B * E] int32
    # a2a transport
    send_dest: Optional[torch.Tensor] = None        # [R, k] position in the owner-major local layout
    send_rows: int = 0
    in_splits: Optional[List[int]] = None
    out_splits: Optional[List[int]] = None


class ExpertParallel:
    def __init__(self, group, device: torch.device, num_experts: int, transport: str = "auto",
                 max_row_bytes: int = 4096, capacity_factor: float = 2.0):
        self.group = group if group is not None else dist.group.WORLD
        self.P = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device
        if num_experts % self.P != 0:
            raise ValueError(f"memory_num_experts={num_experts} is not divisible by the expert-parallel size {self.P}")
        self.E = num_experts
        self.El = num_experts // self.P
        if transport == "auto":
            transport = "peer" if device.type == "cuda" else "a2a"
        self.transport = transport
        self.max_row_bytes = max_row_bytes
        # staging rows per rank = capacity_factor x the balanced load (0 = size for the worst case, P x); a routing
        # that needs more is reported through the kernel status word (code 61), never truncated silently
        self.capacity_factor = float(capacity_factor)
        self.heap = None
        self._recv: List[torch.Tensor] = []
        self._send: List[torch.Tensor] = []
        self._recv_i = 0
        self._send_i = 0
        self._cap_rows = 0
        # tile flow of the fused read (see fused_read): per staging slot, counters of landed rows per tile of the
        # receive buffer and of finished epilogue warps per tile of the send buffer, and how often each send slot
        # has been used that way (its counters only grow)
        self._ready: List[torch.Tensor] = []
        self._done: List[torch.Tensor] = []
        self._done_uses = [0, 0]
        self.wait_limit_ms = 0.0               # 0 = the kernels' own bound (2 s)
        self.fused = os.environ.get("UTTT_B200_EP_FUSED", "1") != "0"

    # ------------------------------------------------------------------ helpers
    def local_experts(self) -> slice:
        return slice(self.rank * self.El, (self.rank + 1) * self.El)

    def gather_sequences(self, t: torch.Tensor) -> torch.Tensor:
        """[B, ...] on every rank -> [P * B, ...] (source-major), differentiable."""
        if self.P == 1:
            return t
        import torch.distributed.nn.functional as dnn
        return torch.cat(dnn.all_gather(t.contiguous(), group=self.group), dim=0)

    def _ensure_heap(self, cap_rows: int) -> None:
        if self.heap is not None:
            if cap_rows > self._cap_rows:
                raise RuntimeError("expert-parallel staging was sized for fewer rows; keep the chunk shape fixed")
            return
        from .symm import SymmetricHeap
        slot = cap_rows * self.max_row_bytes
        self.heap = SymmetricHeap(self.device, self.group,
                                  capacity_bytes=4 * (slot + 4096) + 16 * (cap_rows // TILE + 1024) + (1 << 20))
        self._recv = [self.heap.alloc(slot, torch.uint8) for _ in range(2)]
        self._send = [self.heap.alloc(slot, torch.uint8) for _ in range(2)]
        tiles = cap_rows // TILE
        self._ready = [self.heap.alloc(tiles, torch.int32).zero_() for _ in range(2)]
        self._done = [self.heap.alloc(tiles, torch.int32).zero_() for _ in range(2)]
        self._cap_rows = cap_rows
        self.heap.barrier()

    def _slot(self, pool: List[torch.Tensor], which: str, rows: int, dim: int, dtype: torch.dtype) -> torch.Tensor:
        i = self._recv_i if which == "recv" else self._send_i
        if which == "recv":
            self._recv_i ^= 1
        else:
            self._send_i ^= 1
        item = torch.empty((), dtype=dtype).element_size()
        if dim * item > self.max_row_bytes:
            raise RuntimeError(f"expert-parallel rows of {dim * item} bytes exceed max_row_bytes={self.max_row_bytes}")
        return pool[i][: rows * dim * item].view(dtype).view(rows, dim)

    # ------------------------------------------------------------------ plan
    def plan(self, local: F_ops.GroupPlan, idx: torch.Tensor) -> EPPlan:
        """local: plan of this rank's routed rows over groups b * E + e; idx: [B, N, k] experts."""
        bsz, n, k = idx.shape
        e, p, el = self.E, self.P, self.El
        sizes_all = torch.empty(p, bsz * e, dtype=torch.int32, device=idx.device)
        sizes32 = local.sizes.to(torch.int32).contiguous()
        dist.all_gather_into_tensor(sizes_all.view(-1), sizes32.view(-1), group=self.group)
        g_owner = p * bsz * el
        idx32 = idx.reshape(bsz * n, k).to(torch.int32).contiguous()
        if self.transport == "peer":
            worst = p * bsz * n * k
            want = worst if self.capacity_factor <= 0 else min(worst, int(self.capacity_factor * bsz * n * k))
            cap_rows = ((want + TILE - 1) // TILE + g_owner) * TILE
            self._ensure_heap(cap_rows)
            remote_start, tile_group, offsets, sizes = load(required=True).ep_plan(sizes_all, self.rank, bsz, e,
                                                                                   cap_rows // TILE)
            owner = F_ops.GroupPlan(None, offsets, sizes, tile_group, cap_rows, g_owner, k)
            return EPPlan(local, owner, idx32, sizes32, n, remote_start=remote_start)
        # ---- a2a transport: plain torch, host-visible split sizes
        table = sizes_all.view(p, bsz, p, el).long()                       # [source, b, owner, el]
        padded = (table + TILE - 1) // TILE * TILE
        own = padded[:, :, self.rank, :].reshape(-1)                       # groups (s, b, el) on this owner
        own_sizes = table[:, :, self.rank, :].reshape(-1)
        ends = torch.cumsum(own, 0)
        offsets = torch.cat([ends.new_zeros(1), ends]).to(torch.int32)
        tile_group = torch.repeat_interleave(torch.arange(g_owner, device=idx.device), own // TILE).to(torch.int32)
        rows_owner = int(ends[-1]) if g_owner > 0 else 0
        owner = F_ops.GroupPlan(None, offsets, own_sizes.to(torch.int32), tile_group, rows_owner, g_owner, k)
        # sender side: owner-major order of this rank's groups (owner, b, el)
        mine = padded[self.rank].permute(1, 0, 2).reshape(-1)              # [owner, b, el]
        starts = torch.cumsum(mine, 0) - mine
        b_of = torch.arange(bsz, device=idx.device).repeat_interleave(n).view(-1, 1)
        ex = idx32.long()
        gid2 = (ex // el) * (bsz * el) + b_of * el + ex % el               # [R, k]
        gid1 = b_of * e + ex
        within = local.dest - local.offsets.long()[gid1]
        send_dest = starts[gid2] + within
        per_owner = mine.view(p, -1).sum(1)
        in_splits = [int(v) for v in per_owner.tolist()]
        out_splits = [int(v) for v in padded[:, :, self.rank, :].reshape(p, -1).sum(1).tolist()]
        return EPPlan(local, owner, idx32, sizes32, n, send_dest=send_dest, send_rows=sum(in_splits), in_splits=in_splits,
                      out_splits=out_splits)

    # ------------------------------------------------------------------ dispatch / combine
    def dispatch(self, rows: torch.Tensor, weights: Optional[torch.Tensor], plan: EPPlan) -> torch.Tensor:
        """rows [R, D] (optionally scaled per routed copy by weights [R, k]) -> owner layout [rows_owner, D]."""
        if self.transport == "peer":
            with trace_range("ep.dispatch"):
                return _PeerDispatch.apply(rows, weights, self, plan)
        import torch.distributed.nn.functional as dnn
        r, d = rows.shape
        k = plan.idx.shape[1]
        src = rows.unsqueeze(1).expand(r, k, d)
        if weights is not None:
            src = src * weights.unsqueeze(-1).to(rows.dtype)
        staged = rows.new_zeros(plan.send_rows, d).index_copy(0, plan.send_dest.reshape(-1), src.reshape(r * k, d))
        out = rows.new_empty(sum(plan.out_splits), d)
        return dnn.all_to_all_single(out, staged, plan.out_splits, plan.in_splits, group=self.group)

    def combine(self, yp: torch.Tensor, weights: Optional[torch.Tensor], plan: EPPlan) -> torch.Tensor:
        """Owner layout [rows_owner, D] -> [R, D]: y[r] = sum_j weights[r, j] * (row of copy (r, j))."""
        if self.transport == "peer":
            with trace_range("ep.combine"):
                return _PeerCombine.apply(yp, weights, self, plan)
        import torch.distributed.nn.functional as dnn
        d = yp.shape[1]
        back = yp.new_empty(plan.send_rows, d)
        back = dnn.all_to_all_single(back, yp.contiguous(), plan.in_splits, plan.out_splits, group=self.group)
        picked = back[plan.send_dest]                                       # [R, k, D]
        if weights is not None:
            picked = picked * weights.unsqueeze(-1).to(picked.dtype)
        return picked.sum(1)

    def barrier(self) -> None:
        self.heap.barrier()

    # ------------------------------------------------------------------ fused read (forward only)
    def can_fuse_read(self, rows: torch.Tensor, w02: torch.Tensor, w1: torch.Tensor) -> bool:
        """The tile-driven read serves bf16 rows on the peer transport when autograd does not record (evaluation,
        validation, generation); a recorded forward uses dispatch / combine."""
        return (self.fused and self.transport == "peer" and not torch.is_grad_enabled() and rows.is_cuda
                and w02.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and w02.shape[1] % 256 == 0
                and rows.shape[-1] % 64 == 0)

    def fused_read(self, rows: torch.Tensor, weights: torch.Tensor, w02: torch.Tensor, w1: torch.Tensor,
                   plan: EPPlan) -> torch.Tensor:
        """y[r] = sum_j weights[r, j] * W1_e (silu(W0_e x_r) * W2_e x_r) with the rows travelling tile by tile.

        Four kernels, no host-side ordering between them and no staging copies:
        1. ``ep_push`` stores every routed copy at its place in its owner's receive buffer over NVLink and counts the
           rows that have landed per 128-row tile (in the owner's memory);
        2. the owner's gate|up GEMM (SwiGLU in its epilogue) starts each row tile as soon as its count is complete
           (bounded wait in the TMA producer), while later tiles are still in flight;
        3. the owner's down-projection GEMM writes straight into its send buffer and bumps a per-tile counter from
           every epilogue warp once the warp's rows are in memory;
        4. ``ep_pull`` on the home rank waits (bounded) for the counters of the tiles it reads, loads the rows over
           NVLink, un-permutes and forms the gate-weighted sum.
        A wait that runs out writes the device status word (62 / 63); nothing hangs.
        """
        ext = load(required=True)
        rows = rows.contiguous()
        d = rows.shape[1]
        r_owner = plan.owner.rows_padded
        tiles = r_owner // TILE
        ri, si = self._recv_i, self._send_i
        recv = self._slot(self._recv, "recv", r_owner, d, rows.dtype)
        send = self._slot(self._send, "send", r_owner, d, rows.dtype)
        ready, done = self._ready[ri], self._done[si]
        ext.ep_push(rows, None, *_map_args(plan)[:3], plan.sizes32, plan.remote_start, self.heap.peer_ptrs(recv),
                    self.E, plan.rows_per_batch, r_owner, self.heap.peer_ptrs(ready))
        g = plan.owner.num_groups
        hid = ext.gg_nt_swiglu(recv, w02.reshape(g, w02.shape[-2], d), plan.owner.tile_group, ready[:tiles], TILE,
                               self.wait_limit_ms)
        ready.zero_()           # after the GEMM in stream order; the peers' next stores into this slot come later
        ext.gg_nt(hid, w1.reshape(g, d, w1.shape[-1]), plan.owner.tile_group, send, None, 0, done[:tiles],
                  self.wait_limit_ms)
        self._done_uses[si] += 1
        target = self._done_uses[si] * int(ext.gg_nt_done_per_tile(d))
        return ext.ep_pull(self.heap.peer_ptrs(send), weights, *_map_args(plan), self.E, plan.rows_per_batch, d,
                           rows.dtype, r_owner, self.heap.peer_ptrs(done), target, self.wait_limit_ms)


def _map_args(plan: EPPlan):
    return (plan.idx, plan.local.dest.contiguous(), plan.local.offsets, plan.remote_start)


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, weights, ep: ExpertParallel, plan: EPPlan):
        ext = load(required=True)
        rows = rows.contiguous()
        slot = ep._slot(ep._recv, "recv", plan.owner.rows_padded, rows.shape[1], rows.dtype)
        ext.ep_push(rows, weights, *_map_args(plan)[:3], plan.sizes32, plan.remote_start, ep.heap.peer_ptrs(slot),
                    ep.E, plan.rows_per_batch, plan.owner.rows_padded)
        ep.barrier()
        # The staging slot is reused by the dispatch after next, and callers issue several dispatches in a row
        # before consuming any of them (the write path sends keys, values and learning rates back to back), so the
        # rows always leave the slot, with or without autograd.
        out = slot.clone()
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(rows, weights)
        return out

    @staticmethod
    def backward(ctx, dxp):
        ext = load(required=True)
        ep, plan = ctx.ep, ctx.plan
        rows, weights = ctx.saved_tensors
        dxp = dxp.to(rows.dtype).contiguous()
        slot = ep._slot(ep._send, "send", plan.owner.rows_padded, rows.shape[1], rows.dtype)
        slot.copy_(dxp)
        ep.barrier()
        ptrs = ep.heap.peer_ptrs(slot)
        drows = dweights = None
        if ctx.needs_input_grad[0]:
            drows = ext.ep_pull(ptrs, weights, *_map_args(plan), ep.E, plan.rows_per_batch, rows.shape[1], rows.dtype,
                                plan.owner.rows_padded)
        if weights is not None and ctx.needs_input_grad[1]:
            dweights = ext.ep_pull_dot(rows, ptrs, *_map_args(plan), ep.E, plan.rows_per_batch,
                                       plan.owner.rows_padded).to(weights.dtype)
        return drows, dweights, None, None


class _PeerCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, yp, weights, ep: ExpertParallel, plan: EPPlan):
        ext = load(required=True)
        yp = yp.contiguous()
        slot = ep._slot(ep._send, "send", plan.owner.rows_padded, yp.shape[1], yp.dtype)
        slot.copy_(yp)
        ep.barrier()
        out = ext.ep_pull(ep.heap.peer_ptrs(slot), weights, *_map_args(plan), ep.E, plan.rows_per_batch, yp.shape[1],
                          yp.dtype, plan.owner.rows_padded)
        ctx.ep, ctx.plan = ep, plan
        ctx.save_for_backward(yp, weights)
        return out

    @staticmethod
    def backward(ctx, dy):
        ext = load(required=True)
        ep, plan = ctx.ep, ctx.plan
        yp, weights = ctx.saved_tensors
        dy = dy.to(yp.dtype).contiguous()
        dyp = dweights = None
        if weights is not None and ctx.needs_input_grad[1]:
            slot = ep._slot(ep._send, "send", plan.owner.rows_padded, yp.shape[1], yp.dtype)
            slot.copy_(yp)
            ep.barrier()
            dweights = ext.ep_pull_dot(dy, ep.heap.peer_ptrs(slot), *_map_args(plan), ep.E,
                                       plan.rows_per_batch, plan.owner.rows_padded).to(weights.dtype)
        if ctx.needs_input_grad[0]:
            slot = ep._slot(ep._recv, "recv", plan.owner.rows_padded, yp.shape[1], yp.dtype)
            ext.ep_push(dy, weights, *_map_args(plan)[:3], plan.sizes32, plan.remote_start, ep.heap.peer_ptrs(slot),
                        ep.E, plan.rows_per_batch, plan.owner.rows_padded)
            ep.barrier()
            dyp = slot.clone()
        return dyp, dweights, None, None
