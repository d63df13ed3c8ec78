"""Building blocks shared by the language models: norms, sliding-window attention, gated MLP.

Parameter names mirror the reference so that state dicts are interchangeable
(uttt_llm/flame/custom_models/uttt_moe/ref_base.py:673-747 attention,
:820-859 block, :203-246 low-rank fast-weight init).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor):
        """(x + delta, norm(x + delta)): the residual addition runs inside the norm kernel."""
        return ops.add_rms_norm(x, delta, self.weight, self.eps)


class TokenEmbedding(nn.Embedding):
    """``nn.Embedding`` whose lookup and table gradient run on the gather / scatter-add kernels."""

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        if self.max_norm is not None or self.sparse:
            return super().forward(input_ids)
        return ops.embedding(input_ids, self.weight, self.padding_idx)


class LowRankFastWeight(nn.Module):
    """``W = w_left @ w_right (+ 0.5 * I)``: low-rank parameterisation of the initial fast weights."""

    def __init__(self, num_heads: int, out_features: int, in_features: int, rank: int = 32, init_gain: float = 0.5,
                 add_identity: bool = False):
        super().__init__()
        self.num_heads, self.out_features, self.in_features = num_heads, out_features, in_features
        self.rank, self.init_gain, self.add_identity = rank, init_gain, add_identity
        self.w_left = nn.Parameter(torch.empty(num_heads, out_features, rank))
        self.w_right = nn.Parameter(torch.empty(num_heads, rank, in_features))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.normal_(self.w_left, std=1.0 / math.sqrt(self.rank) * self.init_gain)
        nn.init.normal_(self.w_right, std=1.0 / math.sqrt(self.in_features) * self.init_gain)

    def forward(self) -> torch.Tensor:
        w = self.w_left.float() @ self.w_right.float()
        if self.add_identity:
            eye = torch.eye(self.out_features, self.in_features, device=w.device, dtype=w.dtype)
            w = w + 0.5 * eye.unsqueeze(0)
        return w


class GatedMLP(nn.Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x))."""

    def __init__(self, hidden_size: int, intermediate_size: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # one GEMM for gate|up, fused SwiGLU kernel, one GEMM down
        y02 = ops.stacked_linear(x, self.gate_proj.weight, self.up_proj.weight)
        h = ops.swiglu(y02.view(-1, y02.shape[-1])).view(*x.shape[:-1], -1)
        return ops.linear(h, self.down_proj.weight)


class SlidingWindowAttention(nn.Module):
    """Causal attention over (carried key/value history ++ this chunk) with a left window.

    ``forward`` returns the attention output together with the *pre-rotary* flattened q/k/v
    (shared with the fast-weight memory in ``reuse_kv`` mode) and this chunk's rotated keys
    and values for the next chunk's history.
    """

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_heads
        self.num_kv_heads = config.kv_heads
        self.head_dim = config.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.window_size = config.window_size
        self.rope_theta = float(config.rope_theta) if config.rope_theta else 0.0
        self.q_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=config.qkv_bias)
        self.k_proj = nn.Linear(self.hidden_size, self.kv_dim, bias=config.qkv_bias)
        self.v_proj = nn.Linear(self.hidden_size, self.kv_dim, bias=config.qkv_bias)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False) \
            if config.enable_attention_output_proj else None
        # set by the model around a training forward whose regions are recomputed in backward: the attention output
        # of the first pass (25 MB per chunk at the 760M shape) is kept and handed to the recomputation
        self.reuse_store: Optional[dict] = None

    def history_len(self, chunk: int) -> int:
        """Keys carried between chunks.  A window of W needs W-1 predecessors; W are kept when that makes the
        history a whole number of chunks (the kernel masks by position, so one spare key is harmless and the
        history then needs no copy)."""
        if self.window_size is None:
            return 0
        need = max(self.window_size - 1, 0)
        if need > 0 and self.window_size % chunk == 0:
            return self.window_size
        return need

    def forward(self, x: torch.Tensor, k_hist: Optional[torch.Tensor], v_hist: Optional[torch.Tensor],
                offset: int):
        b, l, _ = x.shape
        # three GEMMs with contiguous outputs (a fused QKV GEMM would hand strided views to every consumer)
        q_flat, k_flat, v_flat = ops.fanout_linear(
            x, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight],
            [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias])
        q = q_flat.reshape(b, l, self.num_heads, self.head_dim)
        k = k_flat.reshape(b, l, self.num_kv_heads, self.head_dim)
        v = v_flat.reshape(b, l, self.num_kv_heads, self.head_dim)
        if self.rope_theta > 0:
            q = ops.rope(q, offset, self.rope_theta)
            k = ops.rope(k, offset, self.rope_theta)
        if k_hist is not None and k_hist.shape[1] > 0:
            full_k = torch.cat([k_hist, k], dim=1)
            full_v = torch.cat([v_hist, v], dim=1)
        else:
            full_k, full_v = k, v
        reuse = None if self.reuse_store is None else (self.reuse_store, offset)
        o = ops.swa_attention(q, full_k, full_v, self.window_size, causal=True, reuse=reuse)
        o = o.reshape(b, l, self.hidden_size)
        if self.o_proj is not None:
            o = ops.linear(o, self.o_proj.weight)
        return o, q_flat, k_flat, v_flat, k, v


def trim_history(k_hist, v_hist, k_new, v_new, keep: Optional[int]):
    """Append this chunk's keys/values to the carried history and keep the last ``keep`` positions."""
    if keep is not None and keep == 0:
        return None, None
    if keep is not None and k_new.shape[1] >= keep:
        # the chunk alone covers the history: no concatenation, no copy when the lengths are equal
        if k_new.shape[1] == keep:
            return k_new, v_new
        return k_new[:, k_new.shape[1] - keep:], v_new[:, v_new.shape[1] - keep:]
    if k_hist is not None and k_hist.shape[1] > 0:
        k_new = torch.cat([k_hist, k_new], dim=1)
        v_new = torch.cat([v_hist, v_new], dim=1)
    if keep is not None and k_new.shape[1] > keep:
        k_new = k_new[:, k_new.shape[1] - keep:]
        v_new = v_new[:, v_new.shape[1] - keep:]
    return k_new, v_new


def inv_softplus(x: float) -> float:
    return x + math.log(-math.expm1(-x))


def init_linear_weights(module: nn.Module, std: float) -> None:
    """Linear/Embedding ~ N(0, std), biases zero, norm weights one (ref_base.py:1030-1048)."""
    for m in module.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, mean=0.0, std=std)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, mean=0.0, std=std)
        elif isinstance(m, (RMSNorm, nn.LayerNorm)):
            if getattr(m, "weight", None) is not None:
                nn.init.ones_(m.weight)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)
