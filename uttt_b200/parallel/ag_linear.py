"""Linear layer whose weight is row-sharded over the ranks of a group, gathered inside the GEMM kernel.

``y = x @ W^T`` with ``W [N, K]`` split into ``P`` row blocks; rank ``r`` owns rows ``[r * N/P, (r + 1) * N/P)``.
Every rank keeps a full-size ``[N, K]`` buffer in the symmetric heap of which only its own rows are authoritative
(they are the parameter); ``ops/csrc/ag_gemm.cu`` pulls the other rows from the peers *while* the tensor cores
already multiply the local rows, in one kernel.  This is the fused counterpart of FSDP's "all-gather the weight,
then call the library GEMM" (parallelize_fla.py:470-571 in the reference sets ``reshard_after_forward="never"``,
so the reference never re-gathers either; this layer serves configurations that shard the weights between uses).

Backward: ``dX = dY @ W`` from the gathered buffer; ``dW`` is reduced to its owner with a reduce-scatter.
The caller must make sure the shards are final on every rank before ``forward`` (e.g. the stream-ordered barrier
at the end of the optimizer step).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops._ext import load


class _AGLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shard, layer: "ShardedWeightLinear"):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = load(required=True).ag_linear(x2, layer.shard_ptrs, layer.rank, layer.w_full, layer.ready,
                                          layer.gather_ctas)
        ctx.layer = layer
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        (x2,) = ctx.saved_tensors
        d2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = dshard = None
        if ctx.needs_input_grad[0]:
            dx = torch.mm(d2, layer.w_full).view(ctx.shape)          # every row was gathered by the forward kernel
        if ctx.needs_input_grad[1]:
            dw = torch.mm(d2.t(), x2)
            dshard = torch.empty_like(layer.shard)
            dist.reduce_scatter_tensor(dshard, dw.contiguous(), group=layer.group)
        return dx, dshard, None


class ShardedWeightLinear(nn.Module):
    def __init__(self, heap, in_features: int, out_features: int, gather_ctas: int = 24):
        super().__init__()
        self.group, self.world, self.rank = heap.group, heap.world, heap.rank
        if out_features % (256 * self.world) != 0 or in_features % 64 != 0:
            raise ValueError("ShardedWeightLinear needs out_features % (256 * ranks) == 0 and in_features % 64 == 0")
        self.in_features, self.out_features = in_features, out_features
        self.gather_ctas = gather_ctas
        self.w_full = heap.alloc(out_features * in_features, torch.bfloat16).view(out_features, in_features)
        rows = out_features // self.world
        self.rows_per_rank = rows
        item = 2
        self.shard_ptrs = [b + r * rows * in_features * item for r, b in enumerate(heap.peer_ptrs(self.w_full))]
        self.ready = torch.zeros(out_features // 256, dtype=torch.int32, device=self.w_full.device)
        # the parameter IS this rank's rows of the full-size buffer
        self.shard = nn.Parameter(self.w_full[self.rank * rows:(self.rank + 1) * rows])
        self.heap = heap

    @torch.no_grad()
    def load_full_weight(self, w: torch.Tensor) -> None:
        """Every rank keeps its own rows of ``w`` [N, K]."""
        rows = self.rows_per_rank
        self.shard.copy_(w[self.rank * rows:(self.rank + 1) * rows].to(self.shard.dtype))
        self.heap.barrier()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features or x.dtype != torch.bfloat16:
            raise ValueError("ShardedWeightLinear takes bf16 inputs of width in_features")
        rows = x.numel() // self.in_features
        if rows % 128 != 0:
            raise ValueError("the number of input rows must be a multiple of 128")
        return _AGLinear.apply(x, self.shard, self)
