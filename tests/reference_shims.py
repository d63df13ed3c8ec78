"""Load the reference's own uTTT-MoE model on a CPU-only machine (for the parity tests).

The reference tree (a verbatim copy under ``baseline/_ref/uttt_llm``, not part of this repository's history) is
imported unmodified.  What cannot run without a GPU is replaced *around* it, before the import:

* ``flash_attn.flash_attn_func``        -> masked softmax attention in the input precision (causal, left window);
* ``fla.modules`` (RMSNorm, GatedMLP, FusedCrossEntropyLoss, FusedLinearCrossEntropyLoss, l2_warp) -> plain PyTorch
  statements of the same modules, with the same parameter names;
* the Triton launcher ``rotary_embedding`` inside the reference's ``rotary.py`` -> the same rotation in PyTorch;
  the cos / sin tables are kept in fp32 (the reference builds them in bf16 on the GPU);
* the Triton grouped kernels (``lact_moe_triton``) are made un-importable, which is the reference's own switch to
  its per-(sequence, expert) loop implementation (modeling_recurrent_lact.py:27-44, 221-261, 389-451).

Everything else - routing, bias handling, learning rates, momentum, Newton-Schulz, renormalisation, the chunk loop,
the backward modes - is the reference's code.  ``load_reference()`` returns the package module or ``None`` when the
tree is absent.
"""
from __future__ import annotations

import importlib
import importlib.machinery
import math
import os
import sys
import types
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

REF_ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "uttt_llm")


# ----------------------------------------------------------------------------- stand-ins
def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), **_):
    """q [B, Lq, H, D], k / v [B, Lk, Hk, D]; queries are the LAST Lq positions of the keys (flash-attn convention)."""
    dt = k.dtype
    b, lq, h, d = q.shape
    lk, hk = k.shape[1], k.shape[2]
    qf, kf, vf = q.to(dt).transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if hk != h:
        kf = kf.repeat_interleave(h // hk, dim=1)
        vf = vf.repeat_interleave(h // hk, dim=1)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    qi = torch.arange(lq, device=q.device).unsqueeze(1) + (lk - lq)
    ki = torch.arange(lk, device=q.device).unsqueeze(0)
    allowed = torch.ones(lq, lk, dtype=torch.bool, device=q.device)
    if causal:
        allowed &= ki <= qi
    left, right = window_size
    if left is not None and left >= 0:
        allowed &= ki >= qi - left
    if right is not None and right >= 0 and not causal:
        allowed &= ki <= qi + right
    s = s.masked_fill(~allowed, float("-inf"))
    o = torch.matmul(torch.softmax(s.float(), dim=-1).to(dt), vf)
    return o.transpose(1, 2).contiguous()


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, elementwise_affine=True, bias=False, eps=1e-5, **_):
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps
        self.weight = nn.Parameter(torch.ones(hidden_size)) if elementwise_affine else None

    def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
        if residual is not None:
            x = x + residual
        y = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.float()
        y = y.to(x.dtype)
        return (y, x) if prenorm else y


class GatedMLP(nn.Module):
    def __init__(self, hidden_size, hidden_ratio=None, intermediate_size=None, hidden_act="swish", fuse_swiglu=True,
                 **_):
        super().__init__()
        if hidden_ratio is None:
            hidden_ratio = 4
        if intermediate_size is None:
            intermediate_size = int(hidden_size * hidden_ratio * 2 / 3)
            intermediate_size = 256 * ((intermediate_size + 256 - 1) // 256)
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x, **_):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class FusedCrossEntropyLoss(nn.CrossEntropyLoss):
    def __init__(self, ignore_index=-100, reduction="mean", inplace_backward=False, **_):
        super().__init__(ignore_index=ignore_index, reduction=reduction)


class FusedLinearCrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index=-100, use_l2warp=False, **_):
        super().__init__()
        self.ignore_index = ignore_index

    def forward(self, x, target, weight, bias=None):
        logits = F.linear(x, weight, bias)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), target.view(-1),
                               ignore_index=self.ignore_index)


def l2_warp(loss, logits, *_, **__):
    return loss


def rotary_embedding(x, cos, sin, interleaved=False, seqlen_offsets=0, cu_seqlens=None, **_):
    """x [B, T, H, D]; cos / sin [S, R/2]: rotate the first R dims (first half / second half pairing)."""
    assert not interleaved and cu_seqlens is None
    t = x.shape[1]
    off = int(seqlen_offsets)
    c = cos[off:off + t].to(x.dtype)[None, :, None, :]
    s = sin[off:off + t].to(x.dtype)[None, :, None, :]
    r = cos.shape[1]
    x1, x2, rest = x[..., :r], x[..., r:2 * r], x[..., 2 * r:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, rest], dim=-1)


# ----------------------------------------------------------------------------- loader
_CACHED = {}


def _stub_modules():
    fa = types.ModuleType("flash_attn")
    fa.flash_attn_func = flash_attn_func
    fla = types.ModuleType("fla")
    fla.__path__ = []
    mods = types.ModuleType("fla.modules")
    mods.__path__ = []
    mods.RMSNorm, mods.GatedMLP = RMSNorm, GatedMLP
    mods.FusedCrossEntropyLoss, mods.FusedLinearCrossEntropyLoss = FusedCrossEntropyLoss, FusedLinearCrossEntropyLoss
    l2w = types.ModuleType("fla.modules.l2warp")
    l2w.l2_warp = l2_warp
    fla.modules = mods
    mods.l2warp = l2w
    # what the reference's rotary.py pulls in for its Triton launcher (never called here)
    ops = types.ModuleType("fla.ops")
    ops.__path__ = []
    ops_utils = types.ModuleType("fla.ops.utils")
    ops_utils.prepare_chunk_indices = lambda *a, **k: None
    utils = types.ModuleType("fla.utils")
    utils.IS_AMD = False
    utils.autotune_cache_kwargs = {}
    utils.get_multiprocessor_count = lambda *a, **k: 1
    utils.input_guard = lambda fn: fn
    fla.ops, fla.utils, ops.utils = ops, utils, ops_utils
    out = {"flash_attn": fa, "fla": fla, "fla.modules": mods, "fla.modules.l2warp": l2w, "fla.ops": ops,
           "fla.ops.utils": ops_utils, "fla.utils": utils}
    for name, m in out.items():
        m.__spec__ = importlib.machinery.ModuleSpec(name, None)
    return out


def load_reference(package: str = "uttt_moe") -> Optional[types.ModuleType]:
    """Import ``flame.custom_models.<package>`` from the reference tree with the CPU stand-ins in place."""
    if package in _CACHED:
        return _CACHED[package]
    if not os.path.isdir(os.path.join(REF_ROOT, "flame", "custom_models", package)):
        return None
    # everything the reference imports from transformers is imported first, while the real packages are visible
    import transformers.generation  # noqa: F401
    import transformers.modeling_outputs  # noqa: F401
    import transformers.modeling_utils  # noqa: F401
    saved = {}
    stubs = _stub_modules()
    pkg_prefix = f"flame.custom_models.{package}"
    # the Triton kernel package must fail to import: `None` in sys.modules makes `import` raise ImportError
    blocked = [f"{pkg_prefix}.lact_moe_triton", f"{pkg_prefix}.lact_moe_triton.triton_permute",
               f"{pkg_prefix}.lact_moe_triton.lact_swiglu_ffn", f"{pkg_prefix}.lact_moe_triton.lact_fw_grad"]
    names = list(stubs) + blocked + ["flame", "flame.custom_models"]
    for name in names:
        saved[name] = sys.modules.get(name, "absent")
    sys.path.insert(0, REF_ROOT)
    try:
        sys.modules.update(stubs)
        for name in blocked:
            sys.modules[name] = None
        for name, path in (("flame", "flame"), ("flame.custom_models", "flame/custom_models")):
            mod = types.ModuleType(name)
            mod.__path__ = [os.path.join(REF_ROOT, path)]
            sys.modules[name] = mod
        mod = importlib.import_module(pkg_prefix)
        rot = importlib.import_module(pkg_prefix + ".rotary")
        rot.rotary_embedding = rotary_embedding
        orig_update = rot.RotaryEmbedding._update_cos_sin_cache

        def fp32_tables(self, seqlen, device=None, dtype=None):
            return orig_update(self, seqlen, device=device, dtype=torch.float32)
        rot.RotaryEmbedding._update_cos_sin_cache = fp32_tables
    finally:
        sys.path.remove(REF_ROOT)
        for name in list(stubs) + blocked:
            if saved[name] == "absent":
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = saved[name]
    _CACHED[package] = mod
    return mod
