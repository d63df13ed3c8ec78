"""Differentiable ops of the framework.

Every function takes ordinary tensors.  CUDA tensors run the hand-written sm_100a kernels
of the in-tree extension (each wrapped in a ``torch.autograd.Function`` whose backward is
again a kernel, or a composition of these same ops so that gradients of gradients work);
CPU tensors run the plain statements in :mod:`uttt_b200.ops.reference`.

The grouped ("expert-major, tile-padded") layout used by the fast-weight ops:
rows routed to (sequence b, expert e) form group ``g = b*E + e``; every group starts on a
multiple of 128 rows and its tail is zero rows, so a 128-row tensor-core tile never
straddles two groups and token reductions need no masking.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import reference as ref
from ._ext import cuda_ext, has

TILE_ROWS = ref.TILE_ROWS

# kernel launch counter (the benchmark reports how many of our kernels ran in the timed region)
_LAUNCHES = 0


def _count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launch_count() -> int:
    """Number of kernels of this extension launched so far in this process."""
    from ._ext import load
    ext = load()
    native = ext.launch_count() if (ext is not None and hasattr(ext, "launch_count")) else 0
    return int(native) + _LAUNCHES


def _kernel(name: str, *tensors):
    """Extension module if kernel ``name`` should serve these tensors, else None."""
    ext = cuda_ext(*tensors)
    if ext is None or not hasattr(ext, name):
        return None
    return ext


# Library / plain-PyTorch stand-ins on the GPU.  Every op falls back to a plain PyTorch (or library) statement when its
# kernel does not cover a shape or dtype; on CPU that is the intended path.  For bf16 tensors on a GPU it means the
# hot path left the kernels of this extension: the fallbacks are counted per op (``library_fallbacks()``), and in
# strict mode (``set_strict(True)`` or ``UTTT_B200_STRICT=1``; ``bench.py`` and the smoke run turn it on) they raise.
class KernelCoverageError(RuntimeError):
    """A bf16 tensor on the GPU reached an op whose kernel does not cover its shape (strict mode)."""


_STRICT = os.environ.get("UTTT_B200_STRICT", "0") == "1"
_FALLBACK_COUNTS = {}


def set_strict(flag: bool) -> None:
    global _STRICT
    _STRICT = bool(flag)


def library_fallbacks() -> dict:
    """How often each op ran as plain PyTorch / a library call on bf16 GPU tensors in this process."""
    return dict(_FALLBACK_COUNTS)


def _note_fallback(op: str, t, why: str = "") -> None:
    if not (torch.is_tensor(t) and t.is_cuda and t.dtype == torch.bfloat16):
        return
    _FALLBACK_COUNTS[op] = _FALLBACK_COUNTS.get(op, 0) + 1
    if _STRICT:
        raise KernelCoverageError(f"{op}: no kernel of this extension covers {tuple(t.shape)} {t.dtype}"
                                  f"{' (' + why + ')' if why else ''}; set UTTT_B200_STRICT=0 to run it as plain PyTorch")


# =========================================================================== norms
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        ext = cuda_ext(x)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, rstd = ext.rms_norm_fwd(x2, weight, float(eps))
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        ext = cuda_ext(x2)
        dx, dw = ext.rms_norm_bwd(dy.reshape(x2.shape).contiguous(), x2, weight, rstd)
        dwo = None if weight is None else dw.to(weight.dtype)
        return dx.view(ctx.shape), dwo, None


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    if _kernel("rms_norm_fwd", x) is not None and x.shape[-1] % 8 == 0:
        return _RMSNorm.apply(x, weight, eps)
    _note_fallback("rms_norm", x)
    return ref.rms_norm(x, weight, eps)


class _RMSNormGated(torch.autograd.Function):
    """``rms_norm(x) * weight * gate[row]`` in one pass; the backward gives the gate's gradient from the same kernel
    that produces the input and weight gradients (no separate multiply, product or row-sum launches)."""

    @staticmethod
    def forward(ctx, x, weight, gate, eps):
        ext = cuda_ext(x)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        g1 = gate.reshape(-1).to(x2.dtype).contiguous()
        y, rstd = ext.rms_norm_gated_fwd(x2, weight, g1, float(eps))
        ctx.save_for_backward(x2, weight, rstd, g1)
        ctx.shape, ctx.gate_shape, ctx.gate_dtype = x.shape, gate.shape, gate.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd, g1 = ctx.saved_tensors
        ext = cuda_ext(x2)
        dx, dw, dg = ext.rms_norm_gated_bwd(dy.reshape(x2.shape).contiguous(), x2, weight, rstd, g1)
        dwo = None if weight is None else dw.to(weight.dtype)
        return dx.view(ctx.shape), dwo, dg.view(ctx.gate_shape).to(ctx.gate_dtype), None


def rms_norm_gated(x: torch.Tensor, weight: Optional[torch.Tensor], gate: torch.Tensor, eps: float = 1e-6):
    """``rms_norm(x, weight) * gate[..., None]`` with one factor per row (``gate.shape == x.shape[:-1]``)."""
    if _kernel("rms_norm_gated_fwd", x) is not None and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096:
        return _RMSNormGated.apply(x, weight, gate, eps)
    return rms_norm(x, weight, eps) * gate.unsqueeze(-1).to(x.dtype)


class _AddRMSNorm(torch.autograd.Function):
    """s = x + delta; y = rms_norm(s) * weight in one kernel; the backward adds the gradient that reached s
    directly inside the norm's backward kernel."""

    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        ext = cuda_ext(x)
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        d2 = delta.reshape(x2.shape).to(x2.dtype).contiguous()
        s, y, rstd = ext.add_rms_norm_fwd(x2, d2, weight, float(eps))
        ctx.save_for_backward(s, weight, rstd)
        ctx.shape = x.shape
        ctx.delta_dtype = delta.dtype
        return s.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, ds, dy):
        s, weight, rstd = ctx.saved_tensors
        ext = cuda_ext(s)
        if dy is None:
            return ds, (None if ds is None else ds.to(ctx.delta_dtype)), None, None
        ds2 = None if ds is None else ds.reshape(s.shape).to(s.dtype).contiguous()
        g, dw = ext.add_rms_norm_bwd(dy.reshape(s.shape).contiguous(), ds2, s, weight, rstd)
        g = g.view(ctx.shape)
        dwo = None if weight is None else dw.to(weight.dtype)
        return g, g.to(ctx.delta_dtype), dwo, None


def add_rms_norm(x: torch.Tensor, delta: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6):
    """Residual addition fused with the norm that follows it: returns (x + delta, rms_norm(x + delta) * weight)."""
    if _kernel("add_rms_norm_fwd", x) is not None and x.shape[-1] % 8 == 0 and x.shape[-1] <= 4096:
        return _AddRMSNorm.apply(x, delta, weight, eps)
    s = x + delta
    return s, ref.rms_norm(s, weight, eps)


def l2_norm(x: torch.Tensor) -> torch.Tensor:
    return ref.l2_norm(x)


# =========================================================================== embedding
class _Embedding(torch.autograd.Function):
    """Row gather; the backward scatter-adds the output gradient into an fp32 table with vector reductions."""

    @staticmethod
    def forward(ctx, ids, table, padding_idx):
        ext = cuda_ext(table)
        ctx.save_for_backward(ids)
        ctx.vocab, ctx.dtype, ctx.padding_idx = table.shape[0], table.dtype, padding_idx
        return ext.embedding_fwd(table.contiguous(), ids)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        ext = cuda_ext(dy)
        g = ext.embedding_bwd(dy, ids, ctx.vocab)
        if ctx.padding_idx is not None:
            g[ctx.padding_idx].zero_()                   # the padding row never trains
        return None, g.to(ctx.dtype), None


def embedding(ids: torch.Tensor, table: torch.Tensor, padding_idx: Optional[int] = None) -> torch.Tensor:
    """table[ids] with the gather / scatter-add kernels on a GPU (ids: integer tensor of any shape)."""
    if _kernel("embedding_fwd", table) is not None and ids.is_cuda and table.shape[1] % 8 == 0 \
            and table.dtype in (torch.bfloat16, torch.float32):
        return _Embedding.apply(ids.long(), table, padding_idx)
    return torch.nn.functional.embedding(ids, table, padding_idx)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    return ref.layer_norm(x, weight, bias, eps)


# =========================================================================== rotary
_ROPE_TABLES = {}


def rope_table(theta: float, dim: int, length: int, device) -> torch.Tensor:
    """[max_len, dim/2, 2] fp32 (cos, sin) table, angles formed in fp64; cached per (theta, dim, device)."""
    key = (float(theta), int(dim), str(device))
    tab = _ROPE_TABLES.get(key)
    if tab is None or tab.shape[0] < length:
        n = max(length, 4096, 0 if tab is None else 2 * tab.shape[0])
        inv = 1.0 / (float(theta) ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        ang = torch.arange(n, dtype=torch.float64)[:, None] * inv[None, :]
        tab = torch.stack([ang.cos(), ang.sin()], dim=-1).float().to(device).contiguous()
        _ROPE_TABLES[key] = tab
    return tab


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, offset, theta, inverse):
        ext = cuda_ext(x)
        ctx.args = (offset, theta, inverse)
        table = rope_table(theta, x.shape[-1], offset + x.shape[1], x.device)
        return ext.rope_fwd(x.contiguous(), table, int(offset), bool(inverse))

    @staticmethod
    def backward(ctx, dy):
        offset, theta, inverse = ctx.args
        return _Rope.apply(dy, offset, theta, not inverse), None, None, None


def rope(x: torch.Tensor, offset: int, theta: float, inverse: bool = False) -> torch.Tensor:
    """Rotary embedding (first-half/second-half pairing) on x: [b, l, nh, hd]."""
    if _kernel("rope_fwd", x) is not None and x.shape[-1] % 2 == 0:
        return _Rope.apply(x, offset, theta, inverse)
    _note_fallback("rope", x)
    return ref.rope(x, offset, theta, inverse)


class _FwQkPrep(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, fw_heads, rope_dim, theta, offset, silu, norm):
        ext = cuda_ext(x)
        b, l, d = x.shape
        xc = x.contiguous()
        table = rope_table(theta, rope_dim, offset + l, x.device) if rope_dim > 0 else x.new_zeros(1, dtype=torch.float32)
        y, inv = ext.fw_qk_prep_fwd(xc.view(b * l, d), scale, shift, table, fw_heads, rope_dim, int(offset),
                                    int(l), bool(silu), {None: 0, "l2": 1, "rms": 2}[norm])
        ctx.save_for_backward(xc, scale, shift, inv)
        ctx.args = (fw_heads, rope_dim, theta, offset, silu, norm)
        return y.view(b, l, d)

    @staticmethod
    def backward(ctx, dy):
        xc, scale, shift, inv = ctx.saved_tensors
        fw_heads, rope_dim, theta, offset, silu, norm = ctx.args
        ext = cuda_ext(xc)
        b, l, d = xc.shape
        table = rope_table(theta, rope_dim, offset + l, xc.device) if rope_dim > 0 else xc.new_zeros(1, dtype=torch.float32)
        dx, dscale, dshift = ext.fw_qk_prep_bwd(dy.contiguous().view(b * l, d), xc.view(b * l, d), scale, shift, inv,
                                                table, fw_heads, rope_dim, int(offset), int(l), bool(silu),
                                                {None: 0, "l2": 1, "rms": 2}[norm])
        ds = None if scale is None else dscale.to(scale.dtype)
        dsh = None if shift is None else dshift.to(shift.dtype)
        return dx.view(b, l, d), ds, dsh, None, None, None, None, None, None


def fw_qk_prep(x, scale, shift, fw_heads: int, rope_dim: int, theta: float, offset: int, silu: bool,
               norm: Optional[str]) -> torch.Tensor:
    """Fused memory q/k preprocessing: affine -> SiLU -> per-head L2/RMS norm -> rotary."""
    d = x.shape[-1]
    ok = (d // fw_heads) % 8 == 0 and (rope_dim == 0 or (rope_dim % 2 == 0 and (d // fw_heads) % rope_dim == 0))
    if _kernel("fw_qk_prep_fwd", x) is not None and ok:
        return _FwQkPrep.apply(x, scale, shift, fw_heads, rope_dim, theta, offset, silu, norm)
    _note_fallback("fw_qk_prep", x)
    return ref.fw_qk_prep(x, scale, shift, fw_heads, rope_dim, theta, offset, silu, norm)


# =========================================================================== attention
class _SWA(torch.autograd.Function):
    """Forward and backward: the tcgen05 sliding-window kernels of this extension."""

    @staticmethod
    def forward(ctx, q, k, v, window, causal, scale, reuse=None):
        ext = cuda_ext(q)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        hit = None
        if reuse is not None:
            # (store, key): the first call under this key keeps its output and log-sum-exp in the store, the second
            # call (the recomputation of a checkpointed region, same inputs) takes them back instead of running the
            # kernel again.  The output is a fraction of the size of what the region would otherwise have to keep.
            store, key = reuse
            hit = store.pop(key, None)
        if hit is not None:
            o, lse = hit
        else:
            o, lse = ext.swa_fwd(q, k, v, int(window or 0), bool(causal), float(scale))
            if reuse is not None:
                store[key] = (o.detach(), lse)        # an alias that never carries autograd history
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (window, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        window, causal, scale = ctx.args
        ext = cuda_ext(q)
        if not hasattr(ext, "swa_bwd"):
            raise RuntimeError("the loaded extension has no swa_bwd: rebuild it (python -m uttt_b200.ops.build)")
        dq, dk, dv = ext.swa_bwd(do.contiguous(), q, k, v, o, lse, int(window or 0), bool(causal), float(scale))
        return dq, dk, dv, None, None, None, None


def swa_attention(q, k, v, window: Optional[int], causal: bool = True, scale: Optional[float] = None, reuse=None):
    """Sliding-window attention; queries are aligned to the last ``lq`` keys.  [b, l, h, hd] layout.
    ``reuse = (dict, key)``: keep the result of the first call under ``key`` for the second one (see ``_SWA``)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if _kernel("swa_fwd", q) is not None and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 96, 128) \
            and q.shape[2] == k.shape[2]:
        return _SWA.apply(q, k, v, window, causal, scale, reuse if torch.is_grad_enabled() else None)
    if q.is_cuda:
        _note_fallback("swa_attention", q, "head dim or head grouping outside the kernel")
        return _sdpa_attention(q, k, v, window, causal, scale)
    return ref.swa_attention(q, k, v, window, causal, scale)


_MASKS = {}


def _flash_attn_func():
    global _FLASH
    if _FLASH is None:
        try:
            from flash_attn import flash_attn_func
            _FLASH = flash_attn_func
        except Exception:
            _FLASH = False
    return _FLASH


_FLASH = None


def _sdpa_attention(q, k, v, window, causal, scale):
    """Library stand-in used only where the hand-written kernel does not cover the shape."""
    fa = _flash_attn_func()
    if fa and q.dtype in (torch.bfloat16, torch.float16) and causal:
        return fa(q, k, v, softmax_scale=scale, causal=True,
                  window_size=(-1, -1) if window is None else (window - 1, 0))
    b, lq, h, hd = q.shape
    lk = k.shape[1]
    if k.shape[2] != h:
        k = k.repeat_interleave(h // k.shape[2], dim=2)
        v = v.repeat_interleave(h // v.shape[2], dim=2)
    mask = None
    if causal:
        key = (lq, lk, window, str(q.device))
        mask = _MASKS.get(key)
        if mask is None:
            qpos = torch.arange(lk - lq, lk, device=q.device)[:, None]
            kpos = torch.arange(lk, device=q.device)[None, :]
            mask = kpos <= qpos
            if window is not None:
                mask = mask & (kpos > qpos - window)
            _MASKS[key] = mask
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                       scale=scale)
    return o.transpose(1, 2).contiguous()


# =========================================================================== routing / grouped layout
@dataclass
class GroupPlan:
    """Expert-major tile-padded layout for one routing decision (built on the device, no host sync)."""
    dest: torch.Tensor          # [R, k] int64: destination row of (row i, choice j)
    offsets: torch.Tensor       # [G+1] int32: padded group starts
    sizes: torch.Tensor         # [G] int32: real rows per group
    tile_group: torch.Tensor    # [T_max] int32: group of tile t, -1 when unused
    rows_padded: int            # static upper bound on padded rows (multiple of 128)
    num_groups: int
    topk: int
    pairs: Optional[tuple] = None   # (entries [tiles, 2], count [1]) of the two-CTA GEMMs, built on first use


def build_group_plan(expert_idx: torch.Tensor, num_experts: int, reuse=None) -> GroupPlan:
    """``reuse = (dict, key)``: the first call under ``key`` keeps its plan, the second one (the recomputation of the
    same region, same routing) takes it back."""
    if reuse is not None and torch.is_grad_enabled():
        store, key = reuse
        hit = store.pop(key, None)
        if hit is not None:
            return hit
        plan = build_group_plan(expert_idx, num_experts)
        store[key] = plan
        return plan
    bsz, n, k = expert_idx.shape
    ext = _kernel("build_group_plan", expert_idx)
    if ext is not None and num_experts <= 256:
        dest, offsets, sizes, tile_group, _ = ext.build_group_plan(expert_idx.to(torch.int32).contiguous(),
                                                                   int(num_experts))
        rows_padded = ((bsz * n * k + TILE_ROWS - 1) // TILE_ROWS + bsz * num_experts) * TILE_ROWS
    else:
        _note_fallback("build_group_plan", None)
        dest, offsets, sizes, tile_group, rows_padded = ref.build_group_plan(expert_idx, num_experts)
    return GroupPlan(dest, offsets, sizes, tile_group, int(rows_padded), bsz * num_experts, k)


# Two-CTA (cta_group::2) variants of the grouped NT / NN products: pairs of 128-row tiles of one group share one
# 256 x 256 MMA with a third less operand traffic per FLOP.  Measured at the benchmark's shapes they do not beat the
# one-CTA kernels (odd tile counts leave a quarter of the pair slots half empty), so they are opt-in:
# ``UTTT_B200_PAIR=1``.
_USE_PAIRS = os.environ.get("UTTT_B200_PAIR", "0") == "1"


def set_cta_pairs(flag: bool) -> None:
    """Switch the grouped NT / NN products between the two-CTA and the one-CTA kernels (both are tested)."""
    global _USE_PAIRS
    _USE_PAIRS = bool(flag)


def _pairs(plan: GroupPlan):
    """Pair plan of ``plan`` (built by one small kernel the first time a GEMM asks for it; no host sync)."""
    if plan.pairs is None:
        ext = cuda_ext(plan.tile_group)
        plan.pairs = tuple(ext.pair_plan(plan.tile_group, plan.offsets, plan.rows_padded // TILE_ROWS))
    return plan.pairs


def _pair_ok(n: int, plan: GroupPlan) -> bool:
    return _USE_PAIRS and n % 128 == 0 and plan.offsets is not None and plan.tile_group.is_cuda


# =========================================================================== dense projections
_FUSED_WGRAD = False


def set_fused_weight_grad(flag: bool) -> None:
    """Let dense projections add their weight gradient into an existing ``.grad`` buffer inside the GEMM
    (and report no gradient to autograd).  Meant for trainers that own persistent ``.grad`` buffers and call
    ``backward()``; leave it off when gradients of weights are requested through ``torch.autograd.grad``."""
    global _FUSED_WGRAD
    _FUSED_WGRAD = bool(flag)


def _fuse_wgrad(w: torch.Tensor, g2: torch.Tensor) -> bool:
    """True when the weight gradient can be accumulated by the GEMM itself into the existing ``.grad`` buffer."""
    return (_FUSED_WGRAD and w.grad is not None and w.grad.dtype == g2.dtype and w.grad.is_contiguous() and w.is_cuda
            and not torch.is_grad_enabled())


# Dense projections on the batched tcgen05 kernel of this extension instead of the library GEMM.  Measured on a B200
# at the block's shapes the own kernel runs at 0.90 to 1.03 of the library's speed, so the library stays the default
# and ``UTTT_B200_DENSE_GEMM=own`` (or :func:`set_dense_gemm`) selects the own kernel.
_DENSE_OWN = os.environ.get("UTTT_B200_DENSE_GEMM", "library") == "own"


def set_dense_gemm(own: bool) -> None:
    global _DENSE_OWN
    _DENSE_OWN = bool(own)


def _dense_own_ok(m: int, k: int, n: int, *tensors) -> bool:
    return (_DENSE_OWN and m % 128 == 0 and k % 64 == 0 and n % 64 == 0
            and all(t.is_cuda and t.dtype == torch.bfloat16 for t in tensors)
            and _kernel("bmm_general", tensors[0]) is not None)


def _mm_nt(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x2 [M, K] @ w [N, K]^T."""
    if _dense_own_ok(x2.shape[0], x2.shape[1], w.shape[0], x2, w):
        return cuda_ext(x2).bmm_general(x2.contiguous()[None], w.contiguous()[None], 0, 1.0, None, 0.0)[0]
    return torch.mm(x2, w.t())


def _mm_nn(g2: torch.Tensor, w: torch.Tensor, addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """g2 [M, N] @ w [N, K] (+ addend)."""
    if _dense_own_ok(g2.shape[0], g2.shape[1], w.shape[1], g2, w) and (addend is None or addend.dtype == g2.dtype):
        return cuda_ext(g2).bmm_general(g2.contiguous()[None], w.contiguous()[None], 1, 1.0,
                                        None if addend is None else addend.contiguous()[None],
                                        0.0 if addend is None else 1.0)[0]
    if addend is None:
        return torch.mm(g2, w)
    return addend.addmm_(g2, w)


def _mm_tn(g2: torch.Tensor, x2: torch.Tensor, acc: Optional[torch.Tensor] = None) -> torch.Tensor:
    """g2 [T, N]^T @ x2 [T, K] -> [N, K]; added into ``acc`` in place when given."""
    if _dense_own_ok(g2.shape[1], g2.shape[0], x2.shape[1], g2, x2) and (acc is None or acc.dtype == g2.dtype):
        out = cuda_ext(g2).bmm_general(g2.contiguous()[None], x2.contiguous()[None], 2, 1.0,
                                       None if acc is None else acc.contiguous()[None], 0.0 if acc is None else 1.0)[0]
        if acc is None:
            return out
        acc.copy_(out)
        return acc
    if acc is None:
        return torch.mm(g2.t(), x2)
    return acc.addmm_(g2.t(), x2)


class _FanoutLinear(torch.autograd.Function):
    """``y_i = x @ W_i^T (+ b_i)`` for several weights reading the same input.

    Backward adds every ``dY_i @ W_i`` into one input-gradient buffer inside the GEMM (beta = 1) instead of
    leaving n - 1 elementwise adds to autograd, and adds ``dY_i^T @ x`` straight into ``W_i.grad`` when that
    buffer already exists (flat gradient buffers of the sharded trainer), returning no weight gradient then."""

    @staticmethod
    def forward(ctx, x, n, *wb):
        ws, bs = wb[:n], wb[n:]
        ctx.save_for_backward(x, *ws)
        ctx.n = n
        ctx.has_bias = [b is not None for b in bs]
        if _DENSE_OWN:
            x2 = x.reshape(-1, x.shape[-1])
            outs = []
            for w, b in zip(ws, bs):
                y = _mm_nt(x2, w)
                outs.append((y if b is None else y + b).view(*x.shape[:-1], w.shape[0]))
            return tuple(outs)
        outs = tuple(torch.nn.functional.linear(x, w, b) for w, b in zip(ws, bs))
        return outs

    @staticmethod
    def backward(ctx, *gys):
        x, *ws = ctx.saved_tensors
        n = ctx.n
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        gws, gbs = [], []
        for i, (w, gy) in enumerate(zip(ws, gys)):
            if gy is None:
                gws.append(None)
                gbs.append(None)
                continue
            g2 = gy.reshape(-1, gy.shape[-1])
            if ctx.needs_input_grad[0]:
                dx = _mm_nn(g2, w, dx)
            if ctx.needs_input_grad[2 + i]:
                if _fuse_wgrad(w, g2):
                    _mm_tn(g2, x2, w.grad)
                    gws.append(None)
                else:
                    gws.append(_mm_tn(g2, x2))
            else:
                gws.append(None)
            gbs.append(g2.sum(0) if (ctx.has_bias[i] and ctx.needs_input_grad[2 + n + i]) else None)
        return (None if dx is None else dx.view_as(x), None, *gws, *gbs)


class _SplitLinear(torch.autograd.Function):
    """``x @ W^T`` with the rows of ``W`` in ``n`` equal blocks, returned as ``n`` contiguous outputs (a fused q|k|v
    projection whose consumers want contiguous q, k and v: slicing one wide output would cost a strided copy per
    slice, and autograd would rebuild the wide gradient by zero-fill and adds).  Backward accumulates the input
    gradient inside the GEMMs and writes each block of the weight gradient in place."""

    @staticmethod
    def forward(ctx, x, w, n):
        ctx.save_for_backward(x, w)
        ctx.n = n
        x2 = x.reshape(-1, x.shape[-1])
        rows = w.shape[0] // n
        return tuple(_mm_nt(x2, w[i * rows:(i + 1) * rows]).view(*x.shape[:-1], rows) for i in range(n))

    @staticmethod
    def backward(ctx, *gys):
        x, w = ctx.saved_tensors
        n = ctx.n
        rows = w.shape[0] // n
        x2 = x.reshape(-1, x.shape[-1])
        fuse = ctx.needs_input_grad[1] and _fuse_wgrad(w, x2)
        dw = None
        if ctx.needs_input_grad[1] and not fuse:
            dw = torch.zeros_like(w) if any(g is None for g in gys) else torch.empty_like(w)
        dx = None
        for i, gy in enumerate(gys):
            if gy is None:
                continue
            g2 = gy.reshape(-1, rows)
            wi = w[i * rows:(i + 1) * rows]
            if ctx.needs_input_grad[0]:
                dx = _mm_nn(g2, wi, dx)
            if fuse:
                w.grad[i * rows:(i + 1) * rows].addmm_(g2.t(), x2)
            elif dw is not None:
                torch.mm(g2.t(), x2, out=dw[i * rows:(i + 1) * rows])
        return (None if dx is None else dx.view_as(x)), dw, None


def split_linear(x: torch.Tensor, weight: torch.Tensor, n: int):
    """``n`` contiguous outputs of ``x @ W^T`` for ``W`` = ``n`` equal row blocks; see ``_SplitLinear``."""
    if not x.is_cuda or weight.shape[0] % n != 0:
        y = torch.nn.functional.linear(x, weight)
        return tuple(t.contiguous() for t in y.chunk(n, dim=-1))
    return _SplitLinear.apply(x, weight, n)


def fanout_linear(x: torch.Tensor, weights, biases=None):
    """Several linear maps of one input; see ``_FanoutLinear``.  Returns a tuple of outputs."""
    weights = list(weights)
    biases = [None] * len(weights) if biases is None else list(biases)
    if not x.is_cuda:
        return tuple(torch.nn.functional.linear(x, w, b) for w, b in zip(weights, biases))
    return _FanoutLinear.apply(x, len(weights), *weights, *biases)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ W^T (+ b)`` with the weight gradient accumulated in the GEMM when ``W.grad`` exists."""
    return fanout_linear(x, [weight], [bias])[0]


def _stacked_view(a: torch.Tensor, b: torch.Tensor):
    """[a; b] as one matrix without a copy when ``b`` directly follows ``a`` in the same storage, else None."""
    if (a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1] and a.is_contiguous() and b.is_contiguous()
            and a.dtype == b.dtype and a.device == b.device
            and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()
            and b.storage_offset() == a.storage_offset() + a.numel()):
        return torch.as_strided(a.detach(), (a.shape[0] + b.shape[0], a.shape[1]), (a.shape[1], 1), a.storage_offset())
    return None


class _StackedLinear(torch.autograd.Function):
    """``x @ [W_a; W_b]^T`` as ONE GEMM.  When the two weights (and their ``.grad`` buffers) are neighbours in a
    flat buffer the stacked operand is a view; otherwise it is concatenated."""

    @staticmethod
    def forward(ctx, x, wa, wb):
        wc = _stacked_view(wa, wb)
        if wc is None:
            wc = torch.cat([wa.detach(), wb.detach()], dim=0)
        ctx.save_for_backward(x, wa, wb)
        if _DENSE_OWN:
            return _mm_nt(x.reshape(-1, x.shape[-1]), wc).view(*x.shape[:-1], wc.shape[0])
        return torch.nn.functional.linear(x, wc)

    @staticmethod
    def backward(ctx, gy):
        x, wa, wb = ctx.saved_tensors
        wc = _stacked_view(wa, wb)
        if wc is None:
            wc = torch.cat([wa.detach(), wb.detach()], dim=0)
        g2 = gy.reshape(-1, gy.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        dx = _mm_nn(g2, wc).view_as(x) if ctx.needs_input_grad[0] else None
        ga = gb = None
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            gc = None
            if wa.grad is not None and wb.grad is not None and _fuse_wgrad(wa, g2) and _fuse_wgrad(wb, g2):
                gc = _stacked_view(wa.grad, wb.grad)
            if gc is not None:
                _mm_tn(g2, x2, gc)
            else:
                full = _mm_tn(g2, x2)
                ga, gb = full[:wa.shape[0]], full[wa.shape[0]:]
        return dx, ga, gb


def stacked_linear(x: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor) -> torch.Tensor:
    """``cat(x @ W_a^T, x @ W_b^T)`` along the last dim, one GEMM."""
    if not x.is_cuda:
        return torch.nn.functional.linear(x, torch.cat([wa, wb], dim=0))
    return _StackedLinear.apply(x, wa, wb)


# =========================================================================== view-synthesis decoder tail
class _PatchDecode(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, target, views, height, width, patch):
        y = y.contiguous()
        rendering, sse = cuda_ext(y).patch_decode_fwd(y, target, int(views), int(height), int(width), int(patch))
        ctx.save_for_backward(rendering, target)
        ctx.patch, ctx.dtype = int(patch), y.dtype
        return rendering, sse

    @staticmethod
    def backward(ctx, g_render, g_sse):
        rendering, target = ctx.saved_tensors
        dy = cuda_ext(rendering).patch_decode_bwd(rendering, target, g_render, g_sse, ctx.patch, ctx.dtype)
        return dy, None, None, None, None, None


def patch_decode(y: torch.Tensor, target: Optional[torch.Tensor], views: int, height: int, width: int, patch: int):
    """Decoder logits [B, V*T, P*P*3] -> (sigmoid image [B, V, 3, H, W] fp32, squared error per view [B, V]).
    Channel order inside a token is (ph, pw, c); ``target`` may be None (then the error sums are zero)."""
    if _kernel("patch_decode_fwd", y) is not None and y.dtype in (torch.bfloat16, torch.float32):
        return _PatchDecode.apply(y, None if target is None else target.float().contiguous(), views, height, width,
                                  patch)
    b = y.shape[0]
    hh, ww = height // patch, width // patch
    r = torch.sigmoid(y.float()).view(b, views, hh, ww, patch, patch, 3).permute(0, 1, 6, 2, 4, 3, 5)
    r = r.reshape(b, views, 3, height, width)
    sse = ((r - target.float()) ** 2).sum(dim=(2, 3, 4)) if target is not None else r.new_zeros(b, views)
    return r, sse


_POOL_MODES = {"restore": 0, "unit": 1, "none": 2}


class _PoolStep(torch.autograd.Function):
    """n = renorm(m + lr * d), w = bf16(n) in one pass; first-order differentiable."""

    @staticmethod
    def forward(ctx, m, d, lr, mode):
        m, d = m.contiguous(), d.contiguous()
        n, w = cuda_ext(m).pool_step_fwd(m, d, float(lr), int(mode))
        ctx.save_for_backward(m, d)
        ctx.args = (float(lr), int(mode))
        return n, w

    @staticmethod
    def backward(ctx, gn, gw):
        m, d = ctx.saved_tensors
        lr, mode = ctx.args
        gm, gd = cuda_ext(m).pool_step_bwd(m, d, gn, gw, lr, mode)
        return gm, gd, None, None


def pool_step(m: torch.Tensor, d: torch.Tensor, lr: float, renorm: str = "restore",
              compute_dtype: torch.dtype = torch.bfloat16):
    """Master step of a fast-weight matrix stack: ``n = renorm(m + lr * d)`` over the last dim, plus the
    compute-dtype copy.  m: fp32 [..., D]; d: same shape.  Returns (n fp32, w compute_dtype)."""
    ext = _kernel("pool_step_fwd", m)
    if ext is not None and m.dtype == torch.float32 and compute_dtype == torch.bfloat16 \
            and d.dtype in (torch.bfloat16, torch.float32) and ext.pool_step_supported(m.shape[-1]):
        return _PoolStep.apply(m, d, lr, _POOL_MODES[renorm])
    n = m + d.float() * lr
    if renorm == "restore":
        n = n / (n.norm(dim=-1, keepdim=True) + 1e-5) * m.norm(dim=-1, keepdim=True)
    elif renorm == "unit":
        n = torch.nn.functional.normalize(n, dim=-1)
    elif renorm != "none":
        raise ValueError(f"unknown renorm {renorm!r}")
    return n, n.to(compute_dtype)


_ROUTER_MODES = {"softmax": 0, "norm_softmax": 1, "norm_relu": 2}


class _Router(torch.autograd.Function):
    """Fused router (logits, softmax or normalised variant, top-k, combine weights, per-sequence probability sums)."""

    @staticmethod
    def forward(ctx, rows, router, bias, topk, rows_per_batch, alpha, bias_in_logits, renorm, mode, rscale, eps,
                reuse=None):
        ext = cuda_ext(rows)
        hit = None
        if reuse is not None:
            # (store, key), as in _SWA: the recomputation of a region takes the routing of its first pass back
            # (a few MB per call) instead of running the router again
            store, key = reuse
            hit = store.pop(key, None)
        if hit is not None:
            idx, w, probs, psum, logits = hit
        else:
            idx, w, probs, psum, logits = ext.router_fwd(rows, router, bias, int(topk), int(rows_per_batch),
                                                         float(alpha), bool(bias_in_logits), bool(renorm), int(mode),
                                                         float(rscale), float(eps))
            if reuse is not None:
                store[key] = (idx.detach(), w.detach(), probs, psum.detach(), logits)
        ctx.save_for_backward(rows, router, probs, idx, logits)
        ctx.args = (int(rows_per_batch), float(alpha), bool(renorm), int(mode), float(rscale), float(eps))
        ctx.mark_non_differentiable(idx)
        return idx, w, psum

    @staticmethod
    def backward(ctx, _gidx, gw, gpsum):
        rows, router, probs, idx, logits = ctx.saved_tensors
        rpb, alpha, renorm, mode, rscale, eps = ctx.args
        ext = cuda_ext(rows)
        drows, drouter = ext.router_bwd(rows, router, probs, idx, gw, gpsum, rpb, alpha, renorm,
                                        bool(ctx.needs_input_grad[0]), mode, rscale, eps, logits if mode else None)
        return ((drows if ctx.needs_input_grad[0] else None), drouter, None, None, None, None, None, None, None, None,
                None, None)


def route_topk(rows, router, bias, topk: int, alpha: float = 1.0, bias_in_logits: bool = False,
               renorm: bool = False, router_type: str = "softmax", router_scale: float = 0.0,
               norm_eps: float = 1e-6, reuse=None):
    """rows [B, N, D], router [E, D], bias [E] or None -> (idx [B, N, k] int, weights [B*N, k] fp32,
    probs_sum [B, E] fp32).  ``router_type``: 'softmax', 'norm_softmax' (softmax of the L2-normalised logits times
    ``router_scale``, sqrt(E) when 0) or 'norm_relu' (their rectified values, normalised to sum 1).  The bias shifts
    selection only unless ``bias_in_logits``."""
    bsz, n, d = rows.shape
    e = router.shape[0]
    rscale = router_scale if router_scale > 0 else math.sqrt(float(e))
    ext = _kernel("router_fwd", rows)
    if ext is not None and ext.router_supported(d, e, topk) and rows.dtype in (torch.bfloat16, torch.float32):
        idx, w, psum = _Router.apply(rows.reshape(bsz * n, d).contiguous(), router.float().contiguous(),
                                     None if bias is None else bias.detach(), topk, n, alpha, bias_in_logits, renorm,
                                     _ROUTER_MODES[router_type], rscale, norm_eps,
                                     reuse if torch.is_grad_enabled() else None)
        return idx.view(bsz, n, topk), w, psum
    _note_fallback("route_topk", rows, "the router kernel wants D % 8 == 0, D <= 512, E % 8 == 0, E <= 64")
    logits = torch.matmul(rows.float(), router.float().t())
    if bias is not None and bias_in_logits:
        logits = logits + bias.view(1, 1, e)
    sel, probs = ref.route_scores(logits, router_type, router_scale, norm_eps)
    scores = sel if (bias is None or bias_in_logits) else sel + bias.view(1, 1, e)
    idx = torch.topk(scores.detach(), k=topk, dim=-1).indices
    picked = probs.gather(-1, idx)
    if renorm:
        picked = picked / picked.sum(dim=-1, keepdim=True).clamp_min(1e-9)
    return idx, (picked * alpha).view(bsz * n, topk), probs.sum(dim=1)


def route_softmax_topk(rows, router, bias, topk: int, alpha: float = 1.0, bias_in_logits: bool = False,
                       renorm: bool = False):
    """The softmax case of :func:`route_topk`."""
    return route_topk(rows, router, bias, topk, alpha, bias_in_logits, renorm)


def _pad_layout(offsets, sizes):
    """(offsets, sizes) as the int32 pair the scatter kernels use to clear only the padding rows, or (None, None)."""
    if offsets is None or sizes is None or offsets.dtype != torch.int32 or not offsets.is_cuda:
        return None, None
    return offsets, (sizes if sizes.dtype == torch.int32 else sizes.to(torch.int32))


class _Permute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, rows_padded, weights, offsets=None, sizes=None):
        ext = cuda_ext(x)
        x = x.contiguous()
        offsets, sizes = _pad_layout(offsets, sizes)
        ctx.save_for_backward(dest, weights, x if weights is not None else None, offsets, sizes)
        return ext.permute_rows(x, dest, int(rows_padded), weights, offsets, sizes)

    @staticmethod
    def backward(ctx, dout):
        dest, weights, x, offsets, sizes = ctx.saved_tensors
        if weights is None:
            return _Unpermute.apply(dout, dest, None, offsets, sizes), None, None, None, None, None
        ext = cuda_ext(dout)
        dout = dout.contiguous()
        dx = ext.unpermute_rows(dout, dest, weights)
        # dw[i, j] = <x[i], dout[dest[i, j]]>  (the scattered gradient this call also produces is not needed)
        _, dw = ext.unpermute_rows_bwd(x, dout, dest, weights, offsets, sizes)
        return dx, None, None, dw.to(weights.dtype), None, None


class _Unpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, dest, weights, offsets=None, sizes=None):
        ext = cuda_ext(y)
        offsets, sizes = _pad_layout(offsets, sizes)
        ctx.save_for_backward(y, dest, weights, offsets, sizes)
        ctx.rows = y.shape[0]
        return ext.unpermute_rows(y.contiguous(), dest, weights)

    @staticmethod
    def backward(ctx, dout):
        y, dest, weights, offsets, sizes = ctx.saved_tensors
        if weights is None:
            return _Permute.apply(dout, dest, ctx.rows, None, offsets, sizes), None, None, None, None
        ext = cuda_ext(y)
        dy, dw = ext.unpermute_rows_bwd(dout.contiguous(), y, dest, weights, offsets, sizes)
        return dy, None, dw.to(weights.dtype), None, None


def permute_rows(x: torch.Tensor, plan: GroupPlan, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """[R, D] token-major rows -> [rows_padded, D] expert-major (each row copied to its top-k groups,
    copy j scaled by ``weights[i, j]`` when given)."""
    if _kernel("permute_rows", x) is not None and x.shape[-1] % 8 == 0:
        return _Permute.apply(x, plan.dest, plan.rows_padded, weights, plan.offsets, plan.sizes)
    if weights is None:
        _note_fallback("permute_rows", x)
        return ref.permute_rows(x, plan.dest, plan.rows_padded)
    k = plan.dest.shape[1]
    scaled = (x.unsqueeze(1).float() * weights.unsqueeze(-1).float()).to(x.dtype).reshape(-1, x.shape[-1])
    out = scaled.new_zeros(plan.rows_padded, x.shape[-1])
    return out.index_copy(0, plan.dest.reshape(-1), scaled)


def unpermute_rows(y: torch.Tensor, plan: GroupPlan, weights: Optional[torch.Tensor]) -> torch.Tensor:
    """Expert-major rows back to token-major, summing the top-k copies with ``weights`` [R, k]."""
    if _kernel("unpermute_rows", y) is not None and y.shape[-1] % 8 == 0:
        return _Unpermute.apply(y, plan.dest, weights, plan.offsets, plan.sizes)
    _note_fallback("unpermute_rows", y)
    return ref.unpermute_rows(y, plan.dest, weights)


# --------------------------------------------------------------------------- grouped GEMMs
def _gg_kernel_ok(*tensors) -> bool:
    return all(t.dtype == torch.bfloat16 for t in tensors) and _kernel("gg_nt", *tensors) is not None


def _gg_dims_ok(k: int, n: int) -> bool:
    return k % 64 == 0 and n % 64 == 0


# --------------------------------------------------------------------------- gradient sinks for shared weights
# A fast-weight bank is read by every layer of a chunk and by every writer of the chunk boundary, so ~2 L weight
# gradients of the full bank size meet at one tensor.  Left to autograd that is ~2 L bank-sized adds per chunk.
# With a sink, every consumer's token-reduction GEMM adds its contribution into ONE buffer inside the GEMM
# epilogue and reports no gradient; the sink node hands the buffer to the producer of the bank.
_GRAD_SINKS = {}


_SINK_BATCH = max(1, min(4, int(os.environ.get("UTTT_B200_SINK_BATCH", "4"))))


def _sink_flush(entry) -> None:
    """Reduce the pending (a, b, offsets) triples of a sink into its buffer in one launch: the buffer is read and
    written once for up to four consumers instead of once per consumer."""
    pending = entry[1]
    if not pending:
        return
    buf = entry[0]
    cuda_ext(buf).gg_tn_multi([p[0] for p in pending], [p[1] for p in pending], [p[2] for p in pending],
                              buf.shape[0], buf.dtype, buf)
    entry[1] = []


class _GradSink(torch.autograd.Function):
    @staticmethod
    def forward(ctx, w):
        ctx.key = w.data_ptr()
        ctx.meta = (w.shape, w.dtype)
        ctx.set_materialize_grads(False)
        _GRAD_SINKS[ctx.key] = [None, []]
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        entry = _GRAD_SINKS.pop(ctx.key, None)
        buf = None if entry is None else entry[0]
        if buf is None:
            return g
        _sink_flush(entry)
        shape, dtype = ctx.meta
        total = buf.view(shape)
        if g is not None:
            total = total + g.float()
        return total.to(dtype)


def grad_sink(w: torch.Tensor) -> torch.Tensor:
    """Mark ``w`` (a tensor consumed by many grouped GEMMs) so that its consumers accumulate their weight
    gradients in one buffer inside their GEMMs.  Identity in value; a no-op off the kernel path."""
    if w.is_cuda and w.requires_grad and torch.is_grad_enabled() and w.dtype == torch.bfloat16 \
            and w.is_contiguous() and _kernel("gg_tn_segments", w) is not None:
        return _GradSink.apply(w)
    return w


def reset_grad_sinks() -> None:
    """Forget sinks whose backward never ran (e.g. a forward pass that was not differentiated) and the cached
    cotangent conversions of the previous step."""
    _GRAD_SINKS.clear()
    _CAST_CACHE.clear()


def _sink_add(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor, plan) -> bool:
    """If ``w`` has a sink: sink[g] += sum_{r in g} a[r]^T b[r] and True; otherwise False.  The addition is queued
    and runs together with those of the next consumers (at most ``_SINK_BATCH`` per launch); the sink's own backward
    flushes what is left."""
    if torch.is_grad_enabled() or not _GRAD_SINKS:
        return False
    entry = _GRAD_SINKS.get(w.data_ptr())
    if entry is None or not _gg_kernel_ok(a, b) or a.shape[1] % 128 != 0 or b.shape[1] % 64 != 0:
        return False
    if entry[0] is None:
        # accumulated in the dtype of the bank (what autograd's own summation would use), at half the traffic of fp32
        entry[0] = torch.zeros(plan.num_groups, a.shape[1], b.shape[1], device=a.device, dtype=w.dtype)
    entry[1].append((a.contiguous(), b.contiguous(), plan.offsets))
    if len(entry[1]) >= _SINK_BATCH:
        _sink_flush(entry)
    return True


class _GGNT(torch.autograd.Function):
    """out[r] = x[r] @ w[g(r)]^T."""

    @staticmethod
    def forward(ctx, x, w, plan):
        ctx.save_for_backward(x, w)
        ctx.plan = plan
        if _pair_ok(w.shape[1], plan):
            return cuda_ext(x).gg_nt_pair(x.contiguous(), w.contiguous(), plan.tile_group, *_pairs(plan))
        return cuda_ext(x).gg_nt(x.contiguous(), w.contiguous(), plan.tile_group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gg_nn(dy, w, ctx.plan)
        if ctx.needs_input_grad[1] and not _sink_add(w, dy, x, ctx.plan):
            dw = gg_tn(dy, x, ctx.plan, w.dtype)
        return dx, dw, None


class _GGNN(torch.autograd.Function):
    """out[r] = x[r] @ w[g(r)]."""

    @staticmethod
    def forward(ctx, x, w, plan):
        ctx.save_for_backward(x, w)
        ctx.plan = plan
        if _pair_ok(w.shape[2], plan):
            return cuda_ext(x).gg_nn_pair(x.contiguous(), w.contiguous(), plan.tile_group, *_pairs(plan))
        return cuda_ext(x).gg_nn(x.contiguous(), w.contiguous(), plan.tile_group)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gg_nt(dy, w, ctx.plan)
        if ctx.needs_input_grad[1] and not _sink_add(w, x, dy, ctx.plan):
            dw = gg_tn(x, dy, ctx.plan, w.dtype)
        return dx, dw, None


class _GGTN(torch.autograd.Function):
    """out[g] = sum over rows of group g of a[r]^T b[r]."""

    @staticmethod
    def forward(ctx, a, b, plan, out_dtype):
        ctx.save_for_backward(a, b)
        ctx.plan = plan
        return cuda_ext(a).gg_tn_segments(a.contiguous(), b.contiguous(), plan.offsets, plan.num_groups, 1,
                                          out_dtype, None)

    @staticmethod
    def backward(ctx, dg):
        a, b = ctx.saved_tensors
        da = db = None
        dgl = dg.to(a.dtype).contiguous()
        if ctx.needs_input_grad[0]:
            da = gg_nt(b, dgl, ctx.plan)
        if ctx.needs_input_grad[1]:
            db = gg_nn(a, dgl, ctx.plan)
        return da, db, None, None


def gg_nt(x, w, plan: GroupPlan):
    """out[r] = x[r] @ w[group(r)]^T;  x [R, K], w [G, N, K] -> [R, N]."""
    if _gg_kernel_ok(x, w) and _gg_dims_ok(x.shape[1], w.shape[1]):
        return _GGNT.apply(x, w, plan)
    _note_fallback("gg_nt", x)
    return ref.gg_nt(x, w, plan.tile_group)


def gg_nn(x, w, plan: GroupPlan):
    """out[r] = x[r] @ w[group(r)];  x [R, K], w [G, K, N] -> [R, N]."""
    if _gg_kernel_ok(x, w) and _gg_dims_ok(x.shape[1], w.shape[2]):
        return _GGNN.apply(x, w, plan)
    _note_fallback("gg_nn", x)
    return ref.gg_nn(x, w, plan.tile_group)


def gg_tn(a, b, plan: GroupPlan, out_dtype: torch.dtype = torch.float32):
    """out[g] = sum_{r in group g} a[r]^T b[r];  a [R, M], b [R, N] -> [G, M, N] (fp32 accumulation)."""
    if _gg_kernel_ok(a, b) and a.shape[1] % 128 == 0 and b.shape[1] % 64 == 0:
        return _GGTN.apply(a, b, plan, out_dtype)
    if _gg_kernel_ok(a, b) and b.shape[1] % 128 == 0 and a.shape[1] % 64 == 0:
        # the kernel wants 128 rows of output per tile: compute the transposed product and view it back
        return _GGTN.apply(b, a, plan, out_dtype).transpose(1, 2)
    _note_fallback("gg_tn", a)
    return ref.gg_tn(a, b, plan.tile_group, plan.num_groups, out_dtype)


# --------------------------------------------------------------------------- fast-weight pointwise
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y02):
        ctx.save_for_backward(y02)
        return cuda_ext(y02).swiglu_fwd(y02.contiguous())

    @staticmethod
    def backward(ctx, dh):
        (y02,) = ctx.saved_tensors
        return _SwiGLUBwd.apply(dh, y02)


class _SwiGLUBwd(torch.autograd.Function):
    """dy02 = d/dy02 <dh, swiglu(y02)>; differentiable once more (needed by the write's outer gradient)."""

    @staticmethod
    def forward(ctx, dh, y02):
        ctx.save_for_backward(dh, y02)
        return cuda_ext(y02).swiglu_bwd(dh.contiguous(), y02.contiguous())

    @staticmethod
    def backward(ctx, g):
        dh, y02 = ctx.saved_tensors
        d_dh, d_y02 = cuda_ext(y02).swiglu_bwd_bwd(g.contiguous(), dh.contiguous(), y02.contiguous())
        return d_dh, d_y02


def swiglu(y02: torch.Tensor) -> torch.Tensor:
    if _kernel("swiglu_fwd", y02) is not None and y02.shape[-1] % 16 == 0:
        return _SwiGLU.apply(y02)
    _note_fallback("swiglu", y02)
    return ref.swiglu(y02)


class _GGSwiGLU(torch.autograd.Function):
    """hid[r] = silu(x[r] W0[g]^T) * (x[r] W2[g]^T) in one grouped GEMM whose epilogue applies the gate, so the
    [rows, 2I] pre-activations never reach memory (the reference's fused read kernel,
    uttt_llm/flame/custom_models/uttt_moe/lact_moe_triton/triton_grouped_swiglu_kernels.py:83-270).  The backward
    recomputes them in tensor memory and emits dh * d swiglu directly (triton_grouped_swiglu_bwd_kernels.py:49-227)."""

    @staticmethod
    def forward(ctx, x, w02, plan):
        x, w02 = x.contiguous(), w02.contiguous()
        ctx.save_for_backward(x, w02)
        ctx.plan = plan
        if _pair_ok(w02.shape[1], plan):
            return cuda_ext(x).gg_nt_swiglu_pair(x, w02, plan.tile_group, *_pairs(plan))
        return cuda_ext(x).gg_nt_swiglu(x, w02, plan.tile_group)

    @staticmethod
    def backward(ctx, dh):
        x, w02 = ctx.saved_tensors
        plan = ctx.plan
        dy02 = _swiglu_bwd_kernel(x, w02, dh.contiguous(), None, plan, False, False)[0]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gg_nn(dy02, w02, plan)
        if ctx.needs_input_grad[1] and not _sink_add(w02, dy02, x, plan):
            dw = gg_tn(dy02, x, plan, w02.dtype)
        return dx, dw, None


def _swiglu_bwd_kernel(x, w02, dh, lr, plan: GroupPlan, want_h: bool, want_y: bool):
    """(dy02 [* lr], hidden [* lr1] or empty, y02 or empty): the SwiGLU derivative applied in the GEMM epilogue."""
    ext = cuda_ext(x)
    if _pair_ok(w02.shape[1], plan):
        return ext.gg_nt_swiglu_bwd_pair(x, w02, dh, lr, plan.tile_group, *_pairs(plan), want_h, want_y)
    return ext.gg_nt_swiglu_bwd(x, w02, dh, lr, plan.tile_group, want_h, want_y)


def _gg_swiglu_ok(x, w02) -> bool:
    return (_gg_kernel_ok(x, w02) and _kernel("gg_nt_swiglu", x) is not None and x.shape[1] % 64 == 0
            and w02.shape[1] % 256 == 0)


def gg_swiglu(x, w02, plan: GroupPlan):
    """Grouped SwiGLU hidden activation: x [R, K], w02 [G, 2I, K] (gate rows, then up rows) -> [R, I]."""
    if _gg_swiglu_ok(x, w02):
        return _GGSwiGLU.apply(x, w02, plan)
    return swiglu(gg_nt(x, w02, plan))


class _FwWritePW(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y02, dh, lr):
        ctx.save_for_backward(y02, dh, lr)
        return tuple(cuda_ext(y02).fw_write_pw_fwd(y02.contiguous(), dh.contiguous(), lr.contiguous()))

    @staticmethod
    def backward(ctx, g_dy02, g_hlr):
        y02, dh, lr = ctx.saved_tensors
        d_y02, d_dh, d_lr = cuda_ext(y02).fw_write_pw_bwd(g_dy02.contiguous(), g_hlr.contiguous(), y02, dh, lr)
        return d_y02, d_dh, d_lr.to(lr.dtype)


def fw_write_pointwise(y02, dh, lr):
    """Inner-gradient pointwise block of the write: returns (dy02*lr, hidden*lr1)."""
    if _kernel("fw_write_pw_fwd", y02) is not None and y02.shape[-1] % 16 == 0:
        return _FwWritePW.apply(y02, dh, lr.float())
    _note_fallback("fw_write_pointwise", y02)
    return ref.fw_write_pointwise(y02, dh, lr)


def _write_inner(kp, vp, lrp, w02, w1, plan, keep_pre: bool):
    """(dy02 * lr, hidden * lr1, y02 or None[, dh]) of the write from permuted keys / values (kernel path only).

    dh = vp W1 is one grouped GEMM; the product kp W02^T stays in tensor memory and its epilogue applies the
    SwiGLU derivative and the per-row learning rates (the reference's three-GEMM kernel with learning rates,
    lact_moe_triton/triton_grouped_swiglu_bwd_with_lr_kernels.py:49-252).  ``keep_pre`` also writes the
    pre-activations, which the gradient-of-gradient pass needs."""
    dh = gg_nn(vp, w1, plan)
    ext = cuda_ext(kp)
    if _gg_swiglu_ok(kp, w02):
        dy02_lr, h_lr, y02 = _swiglu_bwd_kernel(kp.contiguous(), w02.contiguous(), dh, lrp, plan, True, keep_pre)
    else:
        y02 = gg_nt(kp, w02, plan)
        dy02_lr, h_lr = ext.fw_write_pw_fwd(y02, dh, lrp)
    return (dy02_lr, h_lr, y02, dh) if keep_pre else (dy02_lr, h_lr, None)


class _FwWriteGrad(torch.autograd.Function):
    """Inner gradient of the fast-weight write as one autograd node that keeps only its inputs.

    forward : y02 = kp W02^T, dh = vp W1, (dy02*lr, h*lr1) = pointwise, G02 = (dy02*lr)^T kp, G1 = vp^T (h*lr1)
    backward: recomputes y02 / dh, then runs the gradient-of-gradient chain with the same grouped GEMM
    and pointwise kernels, so no [rows, 2I] intermediate outlives the call
    (the reference does the same in FusedLactSwiGLUFFNBwd,
    uttt_llm/flame/custom_models/uttt_moe/lact_moe_triton/lact_fw_grad.py:51-300).
    """

    @staticmethod
    def forward(ctx, kp, vp, lrp, w02, w1, plan):
        ctx.save_for_backward(kp, vp, lrp, w02, w1)
        ctx.plan = plan
        with torch.no_grad():
            dy02_lr, h_lr, _ = _write_inner(kp, vp, lrp, w02, w1, plan, False)
            g02 = gg_tn(dy02_lr, kp, plan)
            g1 = gg_tn(vp, h_lr, plan)
        return g02, g1

    @staticmethod
    def backward(ctx, c02, c1):
        kp, vp, lrp, w02, w1 = ctx.saved_tensors
        plan = ctx.plan
        ext = cuda_ext(kp)
        with torch.no_grad():
            c02 = _cached_cast("c02", c02, kp.dtype)
            c1 = _cached_cast("c1", c1, kp.dtype)
            dy02_lr, h_lr, y02, dh = _write_inner(kp, vp, lrp, w02, w1, plan, True)
            d_dy02 = gg_nt(kp, c02, plan)            # [R, 2I]
            d_kp = gg_nn(dy02_lr, c02, plan)         # [R, D]
            d_vp = gg_nt(h_lr, c1, plan)             # [R, D]
            d_hlr = gg_nn(vp, c1, plan)              # [R, I]
            del dy02_lr, h_lr
            d_y02, d_dh, d_lr = ext.fw_write_pw_bwd(d_dy02, d_hlr, y02, dh, lrp)
            del d_dy02, d_hlr, y02, dh
            d_kp += gg_nn(d_y02, w02, plan)
            d_w02 = None if _sink_add(w02, d_y02, kp, plan) else gg_tn(d_y02, kp, plan, w02.dtype)
            d_vp += gg_nt(d_dh, w1, plan)
            d_w1 = None if _sink_add(w1, vp, d_dh, plan) else gg_tn(vp, d_dh, plan, w1.dtype)
        return d_kp, d_vp, d_lr, d_w02, d_w1, None


_CAST_CACHE = {}


def _cached_cast(slot: str, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``t.to(dtype)`` remembered per slot: the writer layers of one chunk boundary all receive the SAME
    bank-sized cotangent (it passes through the accumulating nodes unchanged), so it is converted once, not L times.
    The source is kept referenced, so an equal address and version mean the same contents."""
    ent = _CAST_CACHE.get(slot)
    if ent is not None and ent[0].data_ptr() == t.data_ptr() and ent[0].shape == t.shape \
            and ent[0]._version == t._version and ent[1].dtype == dtype:
        return ent[1]
    out = t.to(dtype).contiguous()
    _CAST_CACHE[slot] = (t, out)
    return out


def _gg_tn_acc_(a, b, plan: GroupPlan, acc: torch.Tensor) -> None:
    """acc[g] += sum_{r in g} a[r]^T b[r] (fp32, in place; the add happens in the GEMM epilogue)."""
    cuda_ext(a).gg_tn_segments(a.contiguous(), b.contiguous(), plan.offsets, plan.num_groups, 1, torch.float32,
                               acc.view(plan.num_groups, a.shape[1], b.shape[1]))


class WriteStash:
    """Token reductions of several writer layers, added to the fp32 aggregate in ONE launch per matrix.

    Adding one layer's gradient costs a read-modify-write of the whole aggregate (1.2 GB at the benchmark's shapes,
    three times the bytes of the operands), so the reduction ran at the speed of that traffic.  The stash keeps the
    operands of up to ``limit`` layers alive (about 0.9 GB each) and reduces them together: the group's rows of all
    stashed layers form one long reduction, and the aggregate is read and written once per ``limit`` layers."""

    def __init__(self, limit: int = 4):
        self.limit = int(limit)
        self.items = []

    @property
    def pending(self) -> int:
        return len(self.items)

    def add(self, dy02_lr, kp, vp, h_lr, plan: GroupPlan, acc02, acc1) -> None:
        self.items.append((dy02_lr, kp, vp, h_lr, plan.offsets))
        if len(self.items) >= self.limit:
            self.flush(plan.num_groups, acc02, acc1)

    def flush(self, num_groups: int, acc02, acc1) -> None:
        if not self.items:
            return
        ext = cuda_ext(acc02)
        offs = [it[4] for it in self.items]
        m02, n02 = self.items[0][0].shape[1], self.items[0][1].shape[1]
        ext.gg_tn_multi([it[0] for it in self.items], [it[1] for it in self.items], offs, num_groups, torch.float32,
                        acc02.view(num_groups, m02, n02))
        m1, n1 = self.items[0][2].shape[1], self.items[0][3].shape[1]
        ext.gg_tn_multi([it[2] for it in self.items], [it[3] for it in self.items], offs, num_groups, torch.float32,
                        acc1.view(num_groups, m1, n1))
        _count(0)
        self.items = []


class _FwWriteGradAcc(torch.autograd.Function):
    """:class:`_FwWriteGrad` that adds its result into running fp32 sums (the aggregate over writer layers)
    inside the token-reduction GEMM's epilogue instead of materialising per-layer gradients.  With a
    :class:`WriteStash` the reduction is deferred until ``flush`` (or until the stash is full)."""

    @staticmethod
    def forward(ctx, kp, vp, lrp, w02, w1, plan, acc02, acc1, stash=None, flush=True, skip=False):
        ctx.save_for_backward(kp, vp, lrp, w02, w1)
        ctx.plan = plan
        if skip:
            # the sums already hold the result (kept from the first pass over this region): only the node and its
            # saved inputs are wanted
            ctx.mark_dirty(acc02, acc1)
            return acc02, acc1
        with torch.no_grad():
            dy02_lr, h_lr, _ = _write_inner(kp, vp, lrp, w02, w1, plan, False)
            if stash is None:
                _gg_tn_acc_(dy02_lr, kp, plan, acc02)
                _gg_tn_acc_(vp, h_lr, plan, acc1)
            else:
                stash.add(dy02_lr, kp.contiguous(), vp.contiguous(), h_lr, plan, acc02, acc1)
                if flush:
                    stash.flush(plan.num_groups, acc02, acc1)
        ctx.mark_dirty(acc02, acc1)
        return acc02, acc1

    @staticmethod
    def backward(ctx, c02, c1):
        grads = _FwWriteGrad.backward(ctx, c02.reshape(ctx.plan.num_groups, *c02.shape[-2:]),
                                      c1.reshape(ctx.plan.num_groups, *c1.shape[-2:]))
        return (*grads, c02, c1, None, None, None)


def fw_write_grad(kp, vp, lrp, w02, w1, plan: GroupPlan):
    """(G02 [G, 2I, D], G1 [G, D, I]) fp32: lr-weighted inner gradients of the write, from permuted rows.

    kp, vp: [R, D] expert-major keys and (prob-weighted) values; lrp: [R, 3] fp32; w02 [G, 2I, D]; w1 [G, D, I].
    """
    if _fw_write_kernel_ok(kp, vp, w02, w1):
        return _FwWriteGrad.apply(kp, vp, lrp.float().contiguous(), w02, w1, plan)
    y02 = gg_nt(kp, w02, plan)
    dh = gg_nn(vp, w1, plan)
    dy02_lr, h_lr = fw_write_pointwise(y02, dh, lrp)
    return gg_tn(dy02_lr, kp, plan), gg_tn(vp, h_lr, plan)


def _fw_write_kernel_ok(kp, vp, w02, w1) -> bool:
    return (_gg_kernel_ok(kp, vp, w02, w1) and _gg_dims_ok(kp.shape[1], w02.shape[1]) and w02.shape[1] % 256 == 0
            and kp.shape[1] % 128 == 0)


def fw_write_accumulate_skips(acc02: torch.Tensor, w02: torch.Tensor) -> bool:
    """Whether :func:`fw_write_grad_accumulate` runs as the in-place kernel node for these tensors, which is what a
    caller needs to know before it hands over already complete sums with ``skip=True``."""
    return (acc02.is_cuda and acc02.dtype == torch.float32 and w02.dtype == torch.bfloat16
            and _kernel("gg_tn_segments", acc02) is not None and w02.shape[-1] % 128 == 0
            and w02.shape[-2] % 256 == 0)


def write_stash_for(acc02: torch.Tensor) -> Optional[WriteStash]:
    """A stash for the aggregate ``acc02`` when the kernel path will serve it (see :class:`WriteStash`)."""
    limit = int(os.environ.get("UTTT_B200_WRITE_STASH", "4"))
    if limit > 1 and acc02.is_cuda and acc02.dtype == torch.float32 and _kernel("gg_tn_multi", acc02) is not None:
        return WriteStash(min(limit, 4))
    return None


def fw_write_grad_accumulate(kp, vp, lrp, w02, w1, plan: GroupPlan, acc02: torch.Tensor, acc1: torch.Tensor,
                             stash: Optional[WriteStash] = None, flush: bool = True, skip: bool = False):
    """acc02 += G02, acc1 += G1 (see :func:`fw_write_grad`); returns the updated sums.

    On the GPU the sums are updated in place by the GEMM epilogue; elsewhere new tensors are returned.  With a
    ``stash`` the additions of several calls are fused into one launch: the sums are complete only after a call
    with ``flush=True`` (the last writer layer).  ``skip``: the sums are already complete (see
    :func:`fw_write_accumulate_skips`); record the node, do no arithmetic.
    """
    if _fw_write_kernel_ok(kp, vp, w02, w1) and acc02.dtype == torch.float32 and acc02.is_contiguous() \
            and acc1.is_contiguous():
        return _FwWriteGradAcc.apply(kp, vp, lrp.float().contiguous(), w02, w1, plan, acc02, acc1, stash, flush,
                                     skip)
    assert not skip, "skipping is only offered where fw_write_accumulate_skips() says so"
    if stash is not None and stash.pending:
        stash.flush(plan.num_groups, acc02, acc1)
    g02, g1 = fw_write_grad(kp, vp, lrp, w02, w1, plan)
    return acc02 + g02.view_as(acc02), acc1 + g1.view_as(acc1)


# =========================================================================== Newton-Schulz
def newton_schulz(g: torch.Tensor, coeffs=ref.NS5_COEFFS) -> torch.Tensor:
    """Batched Newton-Schulz orthogonalisation (Muon).  g: [b, m, n] -> same shape, bf16 on GPU."""
    ext = _kernel("bmm_general", g)
    if ext is None or g.shape[1] % 128 != 0 or g.shape[2] % 128 != 0:
        _note_fallback("newton_schulz", g)
        return ref.newton_schulz(g, coeffs)
    return _newton_schulz_kernels(g, coeffs)


class _Bmm(torch.autograd.Function):
    """Batched tcgen05 GEMM without materialised transposes.  mode 0: a @ b^T (a [B,M,K], b [B,N,K]);
    mode 1: a @ b (b [B,K,N]); mode 2: a^T @ b (a [B,K,M], b [B,K,N]).  out = alpha * product + beta * d."""

    @staticmethod
    def forward(ctx, a, b, mode, alpha, d, beta):
        a, b = a.contiguous(), b.contiguous()
        ctx.save_for_backward(a, b)
        ctx.mode, ctx.alpha, ctx.beta, ctx.has_d = mode, alpha, beta, d is not None
        return cuda_ext(a).bmm_general(a, b, int(mode), float(alpha), d, float(beta))

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        dc = dc.contiguous()
        al = ctx.alpha
        da = db = None
        if ctx.mode == 0:
            if ctx.needs_input_grad[0]:
                da = _Bmm.apply(dc, b, 1, al, None, 0.0)
            if ctx.needs_input_grad[1]:
                db = _Bmm.apply(dc, a, 2, al, None, 0.0)
        elif ctx.mode == 1:
            if ctx.needs_input_grad[0]:
                da = _Bmm.apply(dc, b, 0, al, None, 0.0)
            if ctx.needs_input_grad[1]:
                db = _Bmm.apply(a, dc, 2, al, None, 0.0)
        else:
            if ctx.needs_input_grad[0]:
                da = _Bmm.apply(b, dc, 0, al, None, 0.0)
            if ctx.needs_input_grad[1]:
                db = _Bmm.apply(a, dc, 1, al, None, 0.0)
        dd = dc * ctx.beta if ctx.has_d else None
        return da, db, None, None, dd, None


def _bmm_shapes_ok(a, b, mode) -> bool:
    m = a.shape[2] if mode == 2 else a.shape[1]
    k = a.shape[1] if mode == 2 else a.shape[2]
    n = b.shape[1] if mode == 0 else b.shape[2]
    return m % 128 == 0 and n % 64 == 0 and k % 64 == 0


def bmm(a, b, mode: int = 0, alpha: float = 1.0, d=None, beta: float = 0.0):
    """alpha * (a @ b^T | a @ b | a^T @ b) + beta * d for mode 0 | 1 | 2, batched over the leading dim."""
    if _kernel("bmm_general", a) is not None and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 \
            and _bmm_shapes_ok(a, b, mode):
        return _Bmm.apply(a, b, mode, alpha, d, beta)
    _note_fallback("bmm", a, "M % 128, N % 64, K % 64")
    if mode == 0:
        out = torch.bmm(a, b.transpose(1, 2))
    elif mode == 1:
        out = torch.bmm(a, b)
    else:
        out = torch.bmm(a.transpose(1, 2), b)
    out = alpha * out
    return out if d is None else out + beta * d


def bmm_nt(a, b, alpha: float = 1.0, d=None, beta: float = 0.0):
    return bmm(a, b, 0, alpha, d, beta)


class _FrobNormalize(torch.autograd.Function):
    """x[b] = g[b] / (|g[b]|_F + eps) in bf16: two kernels (sum of squares; scale + cast) and a two-kernel VJP."""

    @staticmethod
    def forward(ctx, g, eps):
        g = g.contiguous()
        x, sumsq = cuda_ext(g).frob_normalize_fwd(g, float(eps))
        ctx.save_for_backward(g, sumsq)
        ctx.eps = float(eps)
        return x

    @staticmethod
    def backward(ctx, dx):
        g, sumsq = ctx.saved_tensors
        return cuda_ext(g).frob_normalize_bwd(g, sumsq, dx, ctx.eps), None


class _NSIteration(torch.autograd.Function):
    """One Newton-Schulz iteration ``X' = a X + B X`` (wide; ``A = X X^T``) or ``X' = a X + X B`` (tall;
    ``A = X^T X``) with ``B = b A + c A A``, and its hand-written backward: six batched GEMMs whose epilogues add the
    partial gradients as they are formed (``alpha * product + beta * addend``).  Left to autograd the same six products
    are followed by four bank-sized additions and a scaling per iteration."""

    @staticmethod
    def forward(ctx, x, a, b, c, tall):
        ext = cuda_ext(x)
        x = x.contiguous()
        if tall:
            aa = ext.bmm_general(x, x, 2, 1.0, None, 0.0)            # X^T X   [n, n]
            bb = ext.bmm_general(aa, aa, 0, float(c), aa, float(b))  # c A A^T + b A (A symmetric)
            out = ext.bmm_general(x, bb, 1, 1.0, x, float(a))        # X B + a X
        else:
            aa = ext.bmm_general(x, x, 0, 1.0, None, 0.0)            # X X^T   [m, m]
            bb = ext.bmm_general(aa, aa, 0, float(c), aa, float(b))
            out = ext.bmm_general(bb, x, 1, 1.0, x, float(a))        # B X + a X
        _count(0)
        ctx.save_for_backward(x, aa, bb)
        ctx.coef, ctx.tall = (float(a), float(b), float(c)), bool(tall)
        return out

    @staticmethod
    def backward(ctx, g):
        x, aa, bb = ctx.saved_tensors
        a, b, c = ctx.coef
        ext = cuda_ext(x)
        g = g.to(x.dtype).contiguous()
        mm = ext.bmm_general
        if ctx.tall:
            t1 = mm(g, bb, 1, 1.0, g, a)                  # G B + a G            (B symmetric)
            db = mm(x, g, 2, 1.0, None, 0.0)              # X^T G
            u = mm(db, aa, 1, c, db, b)                   # c dB A + b dB
            da = mm(aa, db, 1, c, u, 1.0)                 # c A dB + u
            t2 = mm(x, da, 1, 1.0, t1, 1.0)               # X dA + t1
            dx = mm(x, da, 0, 1.0, t2, 1.0)               # X dA^T + t2
        else:
            t1 = mm(bb, g, 1, 1.0, g, a)                  # B G + a G
            db = mm(g, x, 0, 1.0, None, 0.0)              # G X^T
            u = mm(db, aa, 1, c, db, b)
            da = mm(aa, db, 1, c, u, 1.0)
            t2 = mm(da, x, 1, 1.0, t1, 1.0)               # dA X + t1
            dx = mm(da, x, 2, 1.0, t2, 1.0)               # dA^T X + t2
        return dx, None, None, None, None


_NS_FUSED_BACKWARD = os.environ.get("UTTT_B200_NS_FUSED_BACKWARD", "1") != "0"


def _ns_iteration_ok(x: torch.Tensor, tall: bool) -> bool:
    m, n = x.shape[1], x.shape[2]
    inner = n if tall else m                      # side of the square Gram matrix
    return (_NS_FUSED_BACKWARD and x.dtype == torch.bfloat16 and m % 128 == 0 and n % 128 == 0 and inner % 128 == 0
            and _kernel("bmm_general", x) is not None)


def _newton_schulz_kernels(g, coeffs):
    """Newton-Schulz in the given orientation: wide X iterates with X X^T on the left, tall X with X^T X on the
    right (X p(X^T X) = p(X X^T) X), so no transpose is ever materialised."""
    if _kernel("frob_normalize_fwd", g) is not None and g.dtype in (torch.float32, torch.bfloat16) \
            and (g.size(1) * g.size(2)) % 4 == 0:
        x = _FrobNormalize.apply(g, 1e-7)
    else:
        x = g.to(torch.bfloat16)
        x = (x / (x.float().norm(dim=(1, 2), keepdim=True) + 1e-7).to(torch.bfloat16)).contiguous()
    tall = g.size(1) > g.size(2)
    for a, b, c in coeffs:
        if _ns_iteration_ok(x, tall):
            x = _NSIteration.apply(x, a, b, c, tall)
            continue
        if tall:
            aa = bmm(x, x, 2)                       # X^T X   [n, n]
            bb = bmm(aa, aa, 0, c, aa, b)           # c A A^T + b A (A symmetric)
            x = bmm(x, bb, 1, 1.0, x, a)            # X B + a X
        else:
            aa = bmm(x, x, 0)                       # X X^T   [m, m]
            bb = bmm(aa, aa, 0, c, aa, b)
            x = bmm(bb, x, 1, 1.0, x, a)            # B X + a X
    return x


# =========================================================================== loss
class _LinearCE(torch.autograd.Function):
    """Chunked lm-head + cross-entropy: logits exist only one token-chunk at a time."""

    @staticmethod
    def forward(ctx, h, weight, labels, ignore_index, chunk):
        ext = cuda_ext(h)
        t = h.shape[0]
        n_valid = (labels != ignore_index).sum().clamp_min(1).float()
        loss = torch.zeros((), device=h.device, dtype=torch.float32)
        dh = torch.empty_like(h)
        dw = torch.zeros(weight.shape, device=h.device, dtype=torch.float32)
        wt = weight.to(h.dtype)
        for s in range(0, t, chunk):
            hs = h[s:s + chunk]
            logits = hs @ wt.t()
            # in place: logits <- (softmax - onehot) (unscaled), loss += sum nll
            ext.ce_fwd_bwd_(logits, labels[s:s + chunk].contiguous(), loss, int(ignore_index))
            dh[s:s + chunk] = logits @ wt
            dw.add_((logits.t() @ hs).float())
        ctx.save_for_backward(dh, dw, n_valid)
        ctx.wdtype = weight.dtype
        return loss / n_valid

    @staticmethod
    def backward(ctx, g):
        dh, dw, n_valid = ctx.saved_tensors
        s = g / n_valid
        return dh * s.to(dh.dtype), (dw * s).to(ctx.wdtype), None, None, None


def linear_cross_entropy(h, weight, labels, ignore_index: int = -100, chunk: int = 8192) -> torch.Tensor:
    """Mean token cross-entropy of ``h @ weight.T`` against ``labels`` (no full logits tensor)."""
    if _kernel("ce_fwd_bwd_", h) is not None and h.dtype == torch.bfloat16:
        return _LinearCE.apply(h, weight, labels, ignore_index, chunk)
    return ref.linear_cross_entropy(h, weight, labels, ignore_index, chunk)[0]


# =========================================================================== view synthesis
def plucker_embed(image, fxfycxcy, c2w, is_target, patch: int) -> torch.Tensor:
    """Posed-image tokens: per pixel (ray o, ray d, o x d, rgb*2-1 or 0 for pose-only views), patchified in
    (ph pw c) order -> [b, v, n_patches, patch*patch*12] (bf16 on the GPU kernel path)."""
    ext = _kernel("plucker_embed", image)
    if ext is not None and image.shape[-1] % patch == 0 and image.shape[-2] % patch == 0:
        return ext.plucker_embed(image.float().contiguous(), fxfycxcy.float().contiguous(), c2w.float().contiguous(),
                                 is_target.to(torch.uint8).contiguous(), int(patch))
    _note_fallback("plucker_embed", image)
    return ref.plucker_embed(image, fxfycxcy, c2w, is_target, patch)
