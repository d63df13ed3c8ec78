"""Block stacks of the view-synthesis model whose memory is not an expert pool: the head-wise dense fast-weight family
(TTT-Dense, uTTT-Dense, depth-partitioned uTTT-Dense), the delta-rule baselines (DeltaNet, Gated DeltaNet) and the
key/value-cache transformer.  Module and parameter names are the reference's, so its checkpoints load strictly:

* ``TTTDenseModel`` (uttt_nvs/models/ttt_dense_block.py:96-473): every block owns ``memory.w0/w1/w2 [h, hd, dh]``.
* ``UTTTDenseModel`` (uttt_dense_block.py:39-521): one ``shared_w0/w1/w2`` read by every block; with
  ``aggregate_write`` the blocks' raw gradients are summed and applied once per view, else block after block.
* ``UTTTDensePartitionedModel`` (uttt_dense_partitioned.py:22-212): ``pool_w{0,1,2}_list[p]``, one state per
  contiguous group of ``layers / num_shared_pools`` blocks.
* ``DeltaNetModel`` / ``GatedDeltaNetModel`` (deltanet_block.py:149-639, gated_deltanet_block.py:139-600): a linear
  map ``w [h, dv, dk]`` per block, written per view with the (gated) delta rule averaged over the view's tokens.
* ``TransformerModel`` (transformer_block.py:38-331): attention over a cache of the posed views' keys / values.

All of them walk the same schedule (:class:`ScheduledStack`): every view-chunk is read by all blocks with the current
state; an ``update`` chunk then writes.  The write's target comes from the block's own memory input, or with ``v_gap``
from the output of block ``min(i + v_gap, layers - 1)``.

The fast weights live as fp32 masters plus unit-norm compute copies (bf16 when the activations are bf16 or autocast
is on, else the activation dtype).  The fast-weight GEMMs are batched over (scene, head) through :func:`ops.bmm`
(the tcgen05 batched kernel where the tile rules hold), attention through :func:`ops.swa_attention`.
"""
from __future__ import annotations

import math
from typing import Any, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..ops import reference as ref
from .blocks import MLP as FusedMLP
from .blocks import SelfAttention as FusedSelfAttention


def inv_softplus(x: float) -> float:
    return x + math.log(-math.expm1(-x))


def _compute_dtype(x: torch.Tensor) -> torch.dtype:
    if x.dtype == torch.bfloat16 or torch.is_autocast_enabled(x.device.type):
        return torch.bfloat16
    return x.dtype


def _bmm(a: torch.Tensor, b: torch.Tensor, mode: int, dt: torch.dtype) -> torch.Tensor:
    """[B, H, ., .] x [B, H, ., .] batched over (B, H); mode 0: a b^T, 1: a b, 2: a^T b.  Operands are cast to
    ``dt`` (so the result does not depend on autocast); autocast is off inside."""
    lead = a.shape[:2]
    a3, b3 = a.reshape(-1, *a.shape[2:]).to(dt), b.reshape(-1, *b.shape[2:]).to(dt)
    with torch.autocast(device_type=a.device.type, enabled=False):
        if dt == torch.bfloat16 and a.is_cuda:
            out = ops.bmm(a3, b3, mode)
        elif mode == 0:
            out = torch.bmm(a3, b3.transpose(1, 2))
        elif mode == 1:
            out = torch.bmm(a3, b3)
        else:
            out = torch.bmm(a3.transpose(1, 2), b3)
    return out.view(*lead, *out.shape[1:])


def _orthogonalise(step: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """Five fixed-coefficient Newton-Schulz iterations on every [rows, cols] slice of a [b, h, rows, cols] step, in the
    precision of the compute copies (the tcgen05 batched kernels on a GPU where the tile rules hold)."""
    flat = step.flatten(0, 1)
    if flat.is_cuda:
        return ops.newton_schulz(flat, ref.NS_FIXED_COEFFS).view_as(step)
    return ref.newton_schulz(flat, ref.NS_FIXED_COEFFS, compute_dtype=dt).view_as(step)


def _heads(x: torch.Tensor, h: int) -> torch.Tensor:
    b, l, _ = x.shape
    return x.view(b, l, h, -1).transpose(1, 2)                    # [b, h, l, d]


def _unheads(x: torch.Tensor) -> torch.Tensor:
    b, h, l, d = x.shape
    return x.transpose(1, 2).reshape(b, l, h * d)


def _rms(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), eps=eps)


def _silu_grad(x: torch.Tensor) -> torch.Tensor:
    s = torch.sigmoid(x)
    return s * (1 + x * (1 - s))


class ScheduledStack(nn.Module):
    """Schedule walk shared by the stacks of this module.  Subclasses provide ``blocks`` and

    * ``init_states(batch, like)`` -> list of states, ``state_of(layer)`` -> index into it,
    * ``read_block(block, x, state)`` -> (x_out, memory_in),
    * ``write(states, caches, mask)``: consumes ``caches[i]["xi_memory_in" | "pre_vi" | "xi_out"]``.
    """

    pre_vi_source = "xi_out"          # what a v_gap write takes from the other block

    def _setup(self, layers: int, v_gap: Optional[int]) -> None:
        self.v_gap = v_gap
        self.v_layer_idxs = [max(min(i + v_gap, layers - 1), 0) for i in range(layers)] if v_gap is not None else []
        self.activation_checkpoint = True
        object.__setattr__(self, "_update_mask_callback", None)     # runtime only: not a submodule, not in state_dict

    def set_update_mask_callback(self, fn) -> None:
        """``fn(source_view, start, end, batch_size, patch_count, device, stage="update")`` -> keep mask [B, L]
        multiplied into the learning rates of that view's write (stacks without learning rates ignore it)."""
        object.__setattr__(self, "_update_mask_callback", fn)

    def _ckpt(self, fn, *args):
        if self.activation_checkpoint and torch.is_grad_enabled():
            return checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False)
        return fn(*args)

    def _mask(self, view: int, cfg, x: torch.Tensor) -> Optional[torch.Tensor]:
        fn = self._update_mask_callback
        if fn is None:
            return None
        m = fn(source_view=view, start=cfg.start, end=cfg.end, batch_size=x.shape[0], patch_count=cfg.end - cfg.start,
               device=x.device, stage="update")
        m = torch.as_tensor(m, device=x.device)
        if tuple(m.shape) != (x.shape[0], cfg.end - cfg.start):
            raise ValueError(f"update mask for source view {view} has shape {tuple(m.shape)}, expected "
                             f"{(x.shape[0], cfg.end - cfg.start)}")
        return m

    def state_of(self, layer: int) -> int:
        return layer

    def forward(self, x: torch.Tensor, info) -> Tuple[torch.Tensor, torch.Tensor, List[Any]]:
        states = self.init_states(x.shape[0], x)
        caches = [dict() for _ in self.blocks]
        outputs, view = [], 0
        for cfg in info["ttt_config"]:
            xi = x[:, cfg.start:cfg.end]
            for i, (blk, cache) in enumerate(zip(self.blocks, caches)):
                xi, mem_in = self.read_block(blk, xi, states[self.state_of(i)])
                cache["xi_out"], cache["xi_memory_in"] = xi, mem_in
            if cfg.update:
                for i, cache in enumerate(caches):
                    cache["pre_vi"] = caches[self.v_layer_idxs[i]][self.pre_vi_source] if self.v_gap is not None \
                        else cache["xi_memory_in"]
                self.write(states, caches, self._mask(view, cfg, x))
                view += 1
            outputs.append(xi)
        return torch.cat(outputs, dim=1), x.new_zeros((), dtype=torch.float32), [{}]


# ----------------------------------------------------------------------------------------------------------------
# head-wise dense fast weights
# ----------------------------------------------------------------------------------------------------------------

class HeadwiseMemory(nn.Module):
    """SwiGLU fast weights per head: ``w0, w2 [hd, dh]``, ``w1 [dh, hd]`` for each of ``dim / hd`` heads.

    read:   q = norm(heads(silu(input_proj x)));  y = output_proj(merge(rms((silu(q w0) * (q w2)) w1)))
    write:  k = norm(heads(silu(k_input_proj x))); with target v / L and per-token, per-head rates lr0, lr1, lr2 the
            raw steps are the lr-weighted outer products of the SwiGLU backward through (w0, w1, w2).
    ``norm`` is the unit l2 norm (``l2_norm``) or an RMS norm without weight.  ``own_weights`` adds ``w0, w1, w2``
    as parameters of this module (TTT-Dense); otherwise the stack owns them."""

    def __init__(self, dim: int, fw_head_dim: Optional[int], inter_multi: float, use_muon: bool = True,
                 l2_norm: bool = False, own_weights: bool = False, **_ignored):
        super().__init__()
        self.dim, self.use_muon, self.l2_norm = dim, use_muon, l2_norm
        self.head_dim = dim if fw_head_dim is None else fw_head_dim
        self.num_heads = dim // self.head_dim
        self.inter_dim = int(self.head_dim * inter_multi)
        self.input_proj = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        self.k_input_proj = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        if own_weights:
            self.w0, self.w1, self.w2 = headwise_parameters(self.num_heads, self.head_dim, self.inter_dim)
        self.output_proj = nn.Linear(dim, dim, bias=False)

    def _features(self, proj, x: torch.Tensor) -> torch.Tensor:
        f = _heads(proj(x), self.num_heads)
        return F.normalize(f, dim=-1, eps=1e-5).to(f.dtype) if self.l2_norm else _rms(f)

    def read(self, x: torch.Tensor, fast) -> torch.Tensor:
        w0, w1, w2 = fast
        dt = w0.dtype
        q = self._features(self.input_proj, x)
        hidden = F.silu(_bmm(q, w0, 1, dt)) * _bmm(q, w2, 1, dt)
        y = _rms(_bmm(hidden, w1, 1, dt))
        return self.output_proj(_unheads(y).to(x.dtype))

    def raw_step(self, x: torch.Tensor, target: torch.Tensor, lr: torch.Tensor, fast):
        """(dw0, dw1, dw2) in fp32 from the snapshot ``fast``; nothing is written."""
        w0, w1, w2 = fast
        dt = w0.dtype
        b, l, _ = x.shape
        lr0, lr1, lr2 = lr.view(b, l, self.num_heads, 3).transpose(1, 2).unsqueeze(-1).unbind(dim=3)   # [b, h, l, 1]
        k = self._features(self.k_input_proj, x)
        gate_pre, up = _bmm(k, w0, 1, dt), _bmm(k, w2, 1, dt)
        gate = F.silu(gate_pre)
        hidden = gate * up
        g = _heads(target.float() / l, self.num_heads)
        d_hidden = _bmm(g, w1, 0, dt)
        d_up = d_hidden * gate
        d_gate_pre = (d_hidden * up) * _silu_grad(gate_pre)
        dw1 = _bmm(hidden * lr1, g, 2, dt)
        dw0 = _bmm(k * lr0, d_gate_pre, 2, dt)
        dw2 = _bmm(k * lr2, d_up, 2, dt)
        return dw0.float(), dw1.float(), dw2.float()

    def apply_step(self, step, master, dt: torch.dtype):
        """Optional Newton-Schulz on each step, fp32 add into the masters, new unit-norm compute copies."""
        if self.use_muon:
            step = tuple(_orthogonalise(s, dt) for s in step)
        master = tuple(m + s.float() for m, s in zip(master, step))
        return unit_columns(master, dt), master

    def extra_repr(self) -> str:
        return (f"fw_head_dim: {self.head_dim}, num_heads: {self.num_heads}, inter_dim: {self.inter_dim}, "
                f"use_muon: {self.use_muon}, l2_norm: {self.l2_norm}")


def headwise_parameters(heads: int, head_dim: int, inter: int):
    return (nn.Parameter(torch.randn(heads, head_dim, inter) / math.sqrt(head_dim)),
            nn.Parameter(torch.randn(heads, inter, head_dim) / math.sqrt(inter)),
            nn.Parameter(torch.randn(heads, head_dim, inter) / math.sqrt(head_dim)))


def unit_columns(master, dt: torch.dtype):
    """Compute copies: every ``[., :, j]`` column of the ``[b, h, rows, cols]`` masters scaled to unit length."""
    return tuple(F.normalize(m, dim=2, eps=1e-5).to(dt) for m in master)


def headwise_state(params, batch: int, dt: torch.dtype):
    master = tuple(p.float().unsqueeze(0).repeat(batch, 1, 1, 1) for p in params)
    return [unit_columns(master, dt), master]


class DenseBlock(nn.Module):
    """attention -> head-wise fast-weight memory -> MLP, each pre-normed with a residual; ``to_v`` / ``to_lr`` turn the
    (RMS-normed) write source into the target and the three per-head learning rates."""

    def __init__(self, dim: int, fw_head_dim: Optional[int] = None, attn_head_dim: int = 64, inter_multi: float = 2,
                 fw_inter_multi: float = 2, base_lr: float = 0.01, own_weights: bool = False, **kwargs):
        super().__init__()
        self.dim = dim
        self.ln_attn = nn.RMSNorm(dim, eps=1e-5)
        self.self_attention = FusedSelfAttention(dim, attn_head_dim)
        self.ln_memory = nn.RMSNorm(dim, eps=1e-5)
        self.memory = HeadwiseMemory(dim, fw_head_dim, fw_inter_multi, own_weights=own_weights, **kwargs)
        self.to_v = nn.Sequential(nn.Linear(dim, dim, bias=False), nn.SiLU())
        self.to_lr = nn.Linear(dim, 3 * self.memory.num_heads, bias=False)
        self.base_lr_inv = inv_softplus(base_lr)
        self.ln_mlp = nn.RMSNorm(dim, eps=1e-5)
        self.mlp = FusedMLP(dim, inter_multi)

    def read(self, x, w0, w1, w2):
        x = x + self.self_attention(ops.rms_norm(x, self.ln_attn.weight, 1e-5))
        mem_in = ops.rms_norm(x, self.ln_memory.weight, 1e-5)
        x = x + self.memory.read(mem_in, (w0, w1, w2))
        x = x + self.mlp(ops.rms_norm(x, self.ln_mlp.weight, 1e-5))
        return x, mem_in

    def raw_step(self, mem_in, pre_vi, mask, w0, w1, w2):
        pre_vi = _rms(pre_vi)
        target = self.to_v(pre_vi)
        with torch.autocast(device_type=pre_vi.device.type, enabled=False):
            lr = F.softplus(F.linear(pre_vi.float(), self.to_lr.weight.float()) + self.base_lr_inv)
            if mask is not None:
                lr = lr * mask[..., None].to(lr.dtype)              # one keep decision per patch, all heads and rates
        return self.memory.raw_step(mem_in, target, lr, (w0, w1, w2))


class _DenseStack(ScheduledStack):
    aggregate_write = False

    def read_block(self, blk, x, state):
        return self._ckpt(blk.read, x, *state[0])

    def write(self, states, caches, mask):
        dt = states[0][0][0].dtype
        if self.aggregate_write:
            total = [None] * len(states)
            for i, (blk, cache) in enumerate(zip(self.blocks, caches)):
                s = self.state_of(i)
                step = self._ckpt(blk.raw_step, cache["xi_memory_in"], cache["pre_vi"], mask, *states[s][0])
                total[s] = step if total[s] is None else tuple(a + b for a, b in zip(total[s], step))
            for s, step in enumerate(total):
                if step is not None:
                    states[s][0], states[s][1] = self.blocks[0].memory.apply_step(step, states[s][1], dt)
        else:
            for i, (blk, cache) in enumerate(zip(self.blocks, caches)):
                s = self.state_of(i)
                step = self._ckpt(blk.raw_step, cache["xi_memory_in"], cache["pre_vi"], mask, *states[s][0])
                states[s][0], states[s][1] = blk.memory.apply_step(step, states[s][1], dt)


class TTTDenseModel(_DenseStack):
    """TTT-Dense: every block has its own fast weights."""

    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, **kwargs):
        super().__init__()
        for key in ("aggregate_write", "pool_mode", "num_shared_pools"):
            kwargs.pop(key, None)
        self._setup(layers, v_gap)
        self.blocks = nn.ModuleList([DenseBlock(dim=dim, own_weights=True, **kwargs) for _ in range(layers)])

    def init_states(self, batch, like):
        dt = _compute_dtype(like)
        return [headwise_state((b.memory.w0, b.memory.w1, b.memory.w2), batch, dt) for b in self.blocks]


class UTTTDenseModel(_DenseStack):
    """uTTT-Dense: one set of fast weights for the whole stack."""

    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, fw_head_dim: Optional[int] = None,
                 fw_inter_multi: float = 1, aggregate_write: bool = False, **kwargs):
        super().__init__()
        kwargs.pop("pool_mode", None)
        self._setup(layers, v_gap)
        self.aggregate_write = bool(aggregate_write)
        head_dim = dim if fw_head_dim is None else fw_head_dim
        self.shared_w0, self.shared_w1, self.shared_w2 = headwise_parameters(dim // head_dim, head_dim,
                                                                             int(head_dim * fw_inter_multi))
        self.blocks = nn.ModuleList([DenseBlock(dim=dim, fw_head_dim=fw_head_dim, fw_inter_multi=fw_inter_multi, **kwargs)
                                     for _ in range(layers)])

    def state_of(self, layer: int) -> int:
        return 0

    def init_states(self, batch, like):
        return [headwise_state((self.shared_w0, self.shared_w1, self.shared_w2), batch, _compute_dtype(like))]


class UTTTDensePartitionedModel(_DenseStack):
    """Depth-partitioned uTTT-Dense: ``num_shared_pools`` contiguous groups of blocks, one state per group."""

    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, fw_head_dim: Optional[int] = None,
                 fw_inter_multi: float = 1, num_shared_pools: int = 1, pool_mode: str = "shared",
                 aggregate_write: bool = False, **kwargs):
        super().__init__()
        pools = int(num_shared_pools)
        if pools <= 0:
            raise ValueError("num_shared_pools must be positive.")
        if pool_mode != "shared":
            raise ValueError("the partitioned dense stack only supports pool_mode='shared'.")
        if layers % pools:
            raise ValueError(f"layers ({layers}) must be divisible by num_shared_pools ({pools}).")
        self._setup(layers, v_gap)
        self.aggregate_write, self.num_shared_pools, self.pool_size = bool(aggregate_write), pools, layers // pools
        head_dim = dim if fw_head_dim is None else fw_head_dim
        params = [headwise_parameters(dim // head_dim, head_dim, int(head_dim * fw_inter_multi)) for _ in range(pools)]
        self.pool_w0_list = nn.ParameterList([p[0] for p in params])
        self.pool_w1_list = nn.ParameterList([p[1] for p in params])
        self.pool_w2_list = nn.ParameterList([p[2] for p in params])
        self.blocks = nn.ModuleList([DenseBlock(dim=dim, fw_head_dim=fw_head_dim, fw_inter_multi=fw_inter_multi, **kwargs)
                                     for _ in range(layers)])

    def state_of(self, layer: int) -> int:
        return layer // self.pool_size

    def init_states(self, batch, like):
        dt = _compute_dtype(like)
        return [headwise_state((self.pool_w0_list[p], self.pool_w1_list[p], self.pool_w2_list[p]), batch, dt)
                for p in range(self.num_shared_pools)]


# ----------------------------------------------------------------------------------------------------------------
# delta-rule baselines
# ----------------------------------------------------------------------------------------------------------------

class ShortConvolution(nn.Module):
    """Causal depth-wise convolution along the tokens of a view, optionally followed by SiLU."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = None):
        super().__init__()
        self.conv = nn.Conv1d(hidden_size, hidden_size, kernel_size, groups=hidden_size, padding=kernel_size - 1,
                              bias=bias)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.conv(x.transpose(1, 2))[..., :x.shape[1]].transpose(1, 2)
        return F.silu(y) if self.activation == "silu" else y


class ScaledRMSNorm(nn.Module):
    """RMS norm with a learned scale; with a gate input the result is multiplied by ``silu(gate)``."""

    def __init__(self, size: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(size))

    def forward(self, x: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight
        return y if gate is None else y * F.silu(gate)


class DeltaMemory(nn.Module):
    """A linear fast map ``w [h, dv, dk]`` per head.

    read:   q = norm(act(q_proj x));  y = o_proj(merge(o_norm(q w^T [, gate g_proj x])))
    write:  k = norm(act(k_proj x));  e = v - k w^T;  step = mean over tokens of beta * e (x) k;
            master = [exp(mean g)] * master + step;  compute copy = rows of master at unit length.
    ``beta = sigmoid(b_proj x)`` (times 2 with ``allow_neg_eigval``; ones without ``use_beta``).  The gated variant adds
    the forget gate ``g = -exp(A_log) * softplus(a_proj x + dt_bias)``.  ``act`` is SiLU through an optional short
    causal convolution, or relu / elu+1 / identity; ``norm`` is l2 or sum."""

    def __init__(self, dim: int, fw_num_heads: int = 1, expand_k: float = 1.0, expand_v: float = 1.0,
                 use_beta: bool = True, noise_repeat: int = 1, repeat_function: Optional[str] = None,
                 use_muon: bool = False, conv_size: int = 4, conv_bias: bool = False, qk_activation: str = "silu",
                 qk_norm: str = "l2", use_output_gate: bool = False, allow_neg_eigval: bool = False,
                 use_short_conv: bool = True, norm_eps: float = 1e-5, gated: bool = False):
        super().__init__()
        if qk_activation not in ("silu", "relu", "elu", "identity"):
            raise ValueError(f"Invalid qk_activation: {qk_activation}")
        if qk_norm not in ("l2", "sum"):
            raise ValueError(f"Invalid qk_norm: {qk_norm}")
        if repeat_function not in ("repeat", "linear"):
            raise ValueError(f"Invalid repeat function: {repeat_function}")
        if repeat_function == "linear" and noise_repeat != 1:
            raise ValueError("repeat_function='linear' is only defined for noise_repeat=1")
        h = fw_num_heads
        self.dim, self.fw_num_heads, self.gated, self.use_muon = dim, h, gated, use_muon
        self.qk_activation, self.qk_norm, self.norm_eps = qk_activation, qk_norm, norm_eps
        self.use_beta, self.allow_neg_eigval, self.use_output_gate = use_beta or gated, allow_neg_eigval, use_output_gate
        if gated:
            if dim % h:
                raise ValueError(f"dim ({dim}) must be divisible by fw_num_heads ({h})")
            self.key_dim, self.head_k_dim = dim, dim // h
            self.head_v_dim = int(self.head_k_dim * expand_v)
            self.value_dim = h * self.head_v_dim
        else:
            self.key_dim, self.value_dim = int(dim * expand_k), int(dim * expand_v)
            if self.key_dim % h or self.value_dim % h:
                raise ValueError(f"key_dim ({self.key_dim}) and value_dim ({self.value_dim}) must be divisible by "
                                 f"fw_num_heads ({h})")
            self.head_k_dim, self.head_v_dim = self.key_dim // h, self.value_dim // h
        self.q_proj = nn.Linear(dim, self.key_dim, bias=False)
        self.k_proj = nn.Linear(dim, self.key_dim, bias=False)
        if gated:
            self.a_proj = nn.Linear(dim, h, bias=False)
        if self.use_beta:
            self.b_proj = nn.Linear(dim, h, bias=False)
        if gated:
            self.A_log = nn.Parameter(torch.log(torch.empty(h, dtype=torch.float32).uniform_(0, 16)))
            dt = torch.exp(torch.rand(h) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
            self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
            self.A_log._no_weight_decay = True
            self.dt_bias._no_weight_decay = True
        self.use_short_conv = use_short_conv
        if use_short_conv:
            act = "silu" if qk_activation == "silu" else None
            self.q_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, act)
            self.k_conv1d = ShortConvolution(self.key_dim, conv_size, conv_bias, act)
        self.w = nn.Parameter(torch.randn(h, self.head_v_dim, self.head_k_dim) / math.sqrt(self.head_k_dim))
        if use_output_gate:
            self.g_proj = nn.Linear(dim, self.value_dim, bias=False)
        self.o_norm = ScaledRMSNorm(self.head_v_dim, eps=norm_eps)
        self.o_proj = nn.Linear(self.value_dim, dim, bias=False)

    def init_state(self, batch: int, dt: torch.dtype):
        master = self.w.float().unsqueeze(0).repeat(batch, 1, 1, 1)
        return [F.normalize(master, dim=-1, eps=1e-5).to(dt), master]

    def _features(self, x: torch.Tensor, which: str) -> torch.Tensor:
        f = getattr(self, f"{which}_proj")(x)
        if self.use_short_conv:
            f = getattr(self, f"{which}_conv1d")(f)
        elif self.qk_activation == "silu":
            f = F.silu(f)
        f = _heads(f, self.fw_num_heads)                              # [b, h, l, dk]
        if self.qk_activation == "relu":
            f = f.relu()
        elif self.qk_activation == "elu":
            f = (F.elu(f, 1.0, False) + 1.0).to(f.dtype)
        if self.qk_norm == "l2":
            return F.normalize(f, dim=-1, eps=self.norm_eps)
        return (f / f.sum(-1, keepdim=True)).to(f.dtype)

    def read(self, x: torch.Tensor, fast: torch.Tensor) -> torch.Tensor:
        q = self._features(x, "q")
        y = _bmm(q, fast, 0, fast.dtype).transpose(1, 2)              # [b, l, h, dv]
        gate = self.g_proj(x).view(*y.shape) if self.use_output_gate else None
        y = self.o_norm(y, gate)
        return self.o_proj(y.flatten(2).to(x.dtype))

    def write(self, x: torch.Tensor, target: torch.Tensor, fast: torch.Tensor, master: torch.Tensor):
        b, l, _ = x.shape
        h = self.fw_num_heads
        with torch.autocast(device_type=x.device.type, enabled=False):
            xf = x.float()
            if self.use_beta:
                beta = torch.sigmoid(F.linear(xf, self.b_proj.weight.float()))
                if self.allow_neg_eigval and not self.gated:
                    beta = beta * 2.0
            else:
                beta = xf.new_ones(b, l, h)
            forget = None
            if self.gated:
                g = -self.A_log.float().exp() * F.softplus(F.linear(xf, self.a_proj.weight.float()) + self.dt_bias.float())
                forget = g.mean(dim=1).exp().view(b, h, 1, 1)
        k = self._features(x, "k")
        # repeating the view's tokens ``noise_repeat`` times leaves the token mean of the step unchanged
        err = _heads(target, h).float() - _bmm(k, fast, 0, fast.dtype).float()
        step = _bmm(beta.transpose(1, 2).unsqueeze(-1) * err, k.float(), 2, torch.float32) / l
        if self.use_muon:
            step = _orthogonalise(step, fast.dtype).float()
        master = master + step if forget is None else forget * master + step
        return F.normalize(master, dim=-1, eps=1e-5).to(fast.dtype), master

    def extra_repr(self) -> str:
        return (f"w: {tuple(self.w.shape)}, fw_num_heads: {self.fw_num_heads}, gated: {self.gated}, "
                f"qk_activation: {self.qk_activation}, qk_norm: {self.qk_norm}")


class _BiasedAttention(FusedSelfAttention):
    def __init__(self, dim: int, head_dim: int, bias: bool = False):
        super().__init__(dim, head_dim)
        if bias:
            self.to_qkv = nn.Linear(dim, 3 * dim, bias=True)
            self.to_out = nn.Linear(dim, dim, bias=True)
        self.bias = bias

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.bias:
            return super().forward(x)
        b, l, _ = x.shape
        q, k, v = self.to_qkv(x).view(b, l, 3, -1, self.head_dim).unbind(dim=2)
        o = ops.swa_attention(q.contiguous(), k.contiguous(), v.contiguous(), None, causal=False)
        return self.to_out(o.reshape(b, l, self.dim))


class _BiasedMLP(nn.Module):
    def __init__(self, dim: int, inter_multi: float, bias: bool = False):
        super().__init__()
        inter = int(dim * inter_multi)
        self.gate = nn.Linear(dim, inter, bias=bias)
        self.up = nn.Linear(dim, inter, bias=bias)
        self.down = nn.Linear(inter, dim, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(F.silu(self.gate(x)) * self.up(x))


def _mlp(dim: int, inter_multi: float, bias: bool) -> nn.Module:
    return _BiasedMLP(dim, inter_multi, True) if bias else FusedMLP(dim, inter_multi)


class DeltaBlock(nn.Module):
    def __init__(self, dim: int, attn_head_dim: int = 64, inter_multi: float = 2, bias: bool = False,
                 repeat_function: str = "repeat", noise_repeat: int = 1, norm_eps: float = 1e-5, gated: bool = False,
                 **kwargs):
        super().__init__()
        self.dim, self.norm_eps = dim, norm_eps
        kwargs.setdefault("use_output_gate", True)                 # the block's default; the bare memory's is off
        self.ln_attn = nn.RMSNorm(dim, eps=norm_eps)
        self.self_attention = _BiasedAttention(dim, attn_head_dim, bias)
        self.ln_memory = nn.RMSNorm(dim, eps=norm_eps)
        self.memory = DeltaMemory(dim, repeat_function=repeat_function, noise_repeat=noise_repeat, norm_eps=norm_eps,
                                  gated=gated, **kwargs)
        self.to_v = nn.Linear(dim, self.memory.value_dim * (noise_repeat if repeat_function == "linear" else 1),
                              bias=False)
        self.ln_mlp = nn.RMSNorm(dim, eps=norm_eps)
        self.mlp = _mlp(dim, inter_multi, bias)

    def read(self, x, fast):
        x = x + self.self_attention(ops.rms_norm(x, self.ln_attn.weight, self.norm_eps))
        mem_in = ops.rms_norm(x, self.ln_memory.weight, self.norm_eps)
        x = x + self.memory.read(mem_in, fast)
        x = x + self.mlp(ops.rms_norm(x, self.ln_mlp.weight, self.norm_eps))
        return x, mem_in

    def write(self, mem_in, pre_vi, fast, master):
        return self.memory.write(mem_in, self.to_v(_rms(pre_vi)), fast, master)


class DeltaNetModel(ScheduledStack):
    gated = False

    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, **kwargs):
        super().__init__()
        self._setup(layers, v_gap)
        self.blocks = nn.ModuleList([DeltaBlock(dim=dim, gated=self.gated, **kwargs) for _ in range(layers)])

    def init_states(self, batch, like):
        dt = _compute_dtype(like)
        return [b.memory.init_state(batch, dt) for b in self.blocks]

    def read_block(self, blk, x, state):
        return self._ckpt(blk.read, x, state[0])

    def write(self, states, caches, mask):
        for blk, cache, state in zip(self.blocks, caches, states):
            state[0], state[1] = self._ckpt(blk.write, cache["xi_memory_in"], cache["pre_vi"], state[0], state[1])


class GatedDeltaNetModel(DeltaNetModel):
    gated = True


# ----------------------------------------------------------------------------------------------------------------
# transformer with a key / value cache of the posed views
# ----------------------------------------------------------------------------------------------------------------

_VERSIONS = ("v0", "v1", "v2", "v3", "v4")


class CachedAttention(nn.Module):
    """Queries of the current view attend (no mask) to the cached keys / values followed by the view's own.

    ``transformer_version`` places an extra square projection in front of the q / k / v projections: none (v0); one for
    all three, owned by the block (v1) or by this module (v2); separate ones for q and for k / v, the latter owned by
    the block (v3) or by this module (v4).  The block applies the same k / v-side projection when it writes the cache."""

    def __init__(self, dim: int, head_dim: int, bias: bool = False, transformer_version: Optional[str] = None,
                 qkv_transform: Optional[nn.Module] = None, kv_transform: Optional[nn.Module] = None):
        super().__init__()
        if transformer_version not in _VERSIONS:
            raise ValueError(f"Invalid transformer version: {transformer_version}")
        self.dim, self.head_dim, self.transformer_version = dim, head_dim, transformer_version
        if transformer_version == "v1":
            self.qkv_transform = qkv_transform
        elif transformer_version == "v2":
            self.qkv_transform = nn.Linear(dim, dim, bias=False)
        elif transformer_version in ("v3", "v4"):
            self.q_transform = nn.Linear(dim, dim, bias=False)
            self.kv_transform = kv_transform if transformer_version == "v3" else nn.Linear(dim, dim, bias=False)
        self.to_q = nn.Linear(dim, dim, bias=bias)
        self.to_kv = nn.Linear(dim, 2 * dim, bias=bias)
        self.to_out = nn.Linear(dim, dim, bias=bias)

    def split_kv(self, kv: torch.Tensor):
        b, l, _ = kv.shape
        k, v = kv.view(b, l, 2, -1, self.head_dim).unbind(dim=2)
        return k.contiguous(), v.contiguous()

    def forward(self, x: torch.Tensor, k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor]) -> torch.Tensor:
        ver = self.transformer_version
        if ver in ("v1", "v2"):
            x_q = x_kv = self.qkv_transform(x)
        elif ver in ("v3", "v4"):
            x_q, x_kv = self.q_transform(x), self.kv_transform(x)
        else:
            x_q = x_kv = x
        b, l, _ = x.shape
        q = self.to_q(x_q).view(b, l, -1, self.head_dim)
        k, v = self.split_kv(self.to_kv(x_kv))
        if k_cache is not None:
            k, v = torch.cat([k_cache.to(k.dtype), k], dim=1), torch.cat([v_cache.to(v.dtype), v], dim=1)
        o = ops.swa_attention(q, k, v, None, causal=False)
        return self.to_out(o.reshape(b, l, self.dim))


class TransformerBlock(nn.Module):
    def __init__(self, dim: int, attn_head_dim: int = 64, bias: bool = False, vi_rms_norm: bool = False,
                 inter_multi: float = 2, transformer_version: Optional[str] = None):
        super().__init__()
        if transformer_version not in _VERSIONS:
            raise ValueError(f"Invalid transformer version: {transformer_version}")
        self.dim, self.head_dim, self.vi_rms_norm, self.transformer_version = dim, attn_head_dim, vi_rms_norm, \
            transformer_version
        self.ln_attn = nn.RMSNorm(dim, eps=1e-5)
        extra = {}
        if transformer_version in ("v1", "v2"):
            self.qkv_transform = nn.Linear(dim, dim, bias=False)
            if transformer_version == "v1":
                extra["qkv_transform"] = self.qkv_transform
        elif transformer_version in ("v3", "v4"):
            self.kv_transform = nn.Linear(dim, dim, bias=False)
            if transformer_version == "v3":
                extra["kv_transform"] = self.kv_transform
        self.self_attention = CachedAttention(dim, attn_head_dim, bias, transformer_version, **extra)
        self.ln_mlp = nn.RMSNorm(dim, eps=1e-5)
        self.mlp = _mlp(dim, inter_multi, bias)

    def read(self, x, k_cache, v_cache):
        mem_in = ops.rms_norm(x, self.ln_attn.weight, 1e-5)
        x = x + self.self_attention(mem_in, k_cache, v_cache)
        x = x + self.mlp(ops.rms_norm(x, self.ln_mlp.weight, 1e-5))
        return x, mem_in

    def cache_entry(self, pre_vi: torch.Tensor, to_kv: Optional[nn.Module]):
        """Keys / values that a posed view leaves in this block's cache.  They are projected from the write source
        with the block-level transform (v1, v2: ``qkv_transform``; v3, v4: ``kv_transform``) and ``to_kv``, which is
        this block's own or the one handed in (the last block's, or the stack's separate one)."""
        if self.vi_rms_norm:
            pre_vi = _rms(pre_vi)
        if self.transformer_version in ("v1", "v2"):
            pre_vi = self.qkv_transform(pre_vi)
        elif self.transformer_version in ("v3", "v4"):
            pre_vi = self.kv_transform(pre_vi)
        return self.self_attention.split_kv((to_kv or self.self_attention.to_kv)(pre_vi))


class TransformerModel(ScheduledStack):
    def __init__(self, layers: int, dim: int, v_gap: Optional[int] = None, pre_vi_source: str = "xi_memory_in",
                 use_separate_last_to_kv: Optional[bool] = None, to_kv_mode: Optional[str] = None, **kwargs):
        super().__init__()
        self._setup(layers, v_gap)
        self.pre_vi_source = pre_vi_source
        if to_kv_mode is None:                                      # the older boolean spelling of the same choice
            to_kv_mode = "separate" if use_separate_last_to_kv else "shared_last"
        if to_kv_mode not in ("separate", "shared_last", "per_layer"):
            raise ValueError(f"Invalid to_kv_mode: {to_kv_mode}")
        self.to_kv_mode = to_kv_mode
        if to_kv_mode == "separate":
            self.last_to_kv = nn.Linear(dim, 2 * dim, bias=False)
        self.blocks = nn.ModuleList([TransformerBlock(dim=dim, **kwargs) for _ in range(layers)])

    def init_states(self, batch, like):
        return [[None, None] for _ in self.blocks]

    def read_block(self, blk, x, state):
        if state[0] is None:
            return self._ckpt(lambda t: blk.read(t, None, None), x)
        return self._ckpt(blk.read, x, state[0], state[1])

    def write(self, states, caches, mask):
        to_kv = {"separate": getattr(self, "last_to_kv", None), "shared_last": self.blocks[-1].self_attention.to_kv,
                 "per_layer": None}[self.to_kv_mode]
        for blk, cache, state in zip(self.blocks, caches, states):
            k, v = blk.cache_entry(cache["pre_vi"], to_kv)
            state[0] = k if state[0] is None else torch.cat([state[0], k.to(state[0].dtype)], dim=1)
            state[1] = v if state[1] is None else torch.cat([state[1], v.to(state[1].dtype)], dim=1)

    def extra_repr(self) -> str:
        return f"pre_vi_source: {self.pre_vi_source}, to_kv_mode: {self.to_kv_mode}"
