"""Plain PyTorch statements of every op in :mod:`uttt_b200.ops`.

These run on any device and dtype, are differentiable through ordinary autograd,
and serve two purposes: they are the CPU path of the framework (fp32 plumbing and
oracle runs), and they are the numerical reference that every CUDA kernel is
tested against.  Nothing here is tuned for speed.

Math sources in the reference implementation:
* RMSNorm / param-free norms .... uttt_llm/flame/custom_models/uttt_moe/ref_base.py:181-195
* rotary (non-interleaved) ...... uttt_llm/flame/custom_models/uttt_moe/rotary.py:15-28
* Newton-Schulz x5 .............. uttt_llm/flame/custom_models/uttt_moe/ttt_operation.py:18-46
* SiLU backprop ................. uttt_llm/flame/custom_models/uttt_moe/ttt_operation.py:4-15
* routing ....................... uttt_llm/flame/custom_models/uttt_moe/moe_routing.py:7-75
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

TILE_ROWS = 128  # row granularity of the grouped layout (one tensor-core M tile)


# --------------------------------------------------------------------------- norms
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def l2_norm(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    return (xf / (xf.norm(dim=-1, keepdim=True) + eps)).to(x.dtype)


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float):
    return F.layer_norm(x.float(), x.shape[-1:], None if weight is None else weight.float(),
                        None if bias is None else bias.float(), eps).to(x.dtype)


# --------------------------------------------------------------------------- rotary
def rope_cos_sin(positions: torch.Tensor, dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = positions.float()[:, None] * inv_freq[None, :]
    return ang.cos(), ang.sin()


def rope(x: torch.Tensor, offset: int, theta: float, inverse: bool = False) -> torch.Tensor:
    """x: [b, l, nh, hd]; rotates (first half, second half) pairs at positions offset..offset+l-1."""
    b, l, nh, hd = x.shape
    pos = torch.arange(offset, offset + l, device=x.device)
    cos, sin = rope_cos_sin(pos, hd, theta)
    if inverse:
        sin = -sin
    cos = cos[None, :, None, :]
    sin = sin[None, :, None, :]
    xf = x.float()
    x1, x2 = xf[..., : hd // 2], xf[..., hd // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def fw_qk_prep(x: torch.Tensor, scale: Optional[torch.Tensor], shift: Optional[torch.Tensor], fw_heads: int,
               rope_dim: int, theta: float, offset: int, silu: bool, norm: Optional[str]) -> torch.Tensor:
    """Memory query/key preprocessing: affine rescale -> SiLU -> per-head norm -> rotary on rope_dim sub-heads.

    x: [b, l, d].  (uttt_llm/flame/custom_models/uttt_moe/modeling_recurrent_lact.py:588-601)
    """
    b, l, d = x.shape
    y = x.float()
    if scale is not None:
        y = y * scale.float() + shift.float()
    if silu:
        y = F.silu(y)
    if norm is not None:
        y = y.view(b, l, fw_heads, d // fw_heads)
        if norm == "l2":
            y = y / (y.norm(dim=-1, keepdim=True) + 1e-5)
        else:
            y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-5)
        y = y.reshape(b, l, d)
    if rope_dim > 0:
        y = rope(y.view(b, l, d // rope_dim, rope_dim), offset, theta).reshape(b, l, d)
    return y.to(x.dtype)


# --------------------------------------------------------------------------- attention
def swa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int], causal: bool = True,
                  scale: Optional[float] = None) -> torch.Tensor:
    """q: [b, lq, h, hd]; k, v: [b, lk, hk, hd] with the queries aligned to the *last* lq keys.

    causal: query i (absolute position lk-lq+i) sees keys j <= its position and, with a
    window W, only j > position - W (itself plus W-1 predecessors).
    """
    b, lq, h, hd = q.shape
    lk, hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if hk != h:
        k = k.repeat_interleave(h // hk, dim=2)
        v = v.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if causal:
        qpos = torch.arange(lk - lq, lk, device=q.device)[:, None]
        kpos = torch.arange(lk, device=q.device)[None, :]
        mask = kpos <= qpos
        if window is not None:
            mask = mask & (kpos > qpos - window)
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(q.dtype)


# --------------------------------------------------------------------------- routing
def route_scores(logits: torch.Tensor, router_type: str, router_scale: float, norm_eps: float):
    """logits: [..., E] fp32 -> (selection_scores, balance_probs)."""
    e = logits.shape[-1]
    if router_type == "softmax":
        return logits, torch.softmax(logits, dim=-1)
    scale = router_scale if router_scale > 0 else math.sqrt(float(e))
    z = logits / logits.norm(dim=-1, keepdim=True).clamp_min(norm_eps)
    if router_type == "norm_softmax":
        sel = z * scale
        return sel, torch.softmax(sel, dim=-1)
    if router_type == "norm_relu":
        sel = F.relu(z) * scale
        ssum = sel.sum(dim=-1, keepdim=True)
        probs = torch.where(ssum > 0, sel / ssum.clamp_min(1e-9), torch.full_like(sel, 1.0 / e))
        return sel, probs
    raise ValueError(f"unknown router_type {router_type!r}")


def build_group_plan(expert_idx: torch.Tensor, num_experts: int):
    """expert_idx: [B, N, k] (int) -> padded expert-major layout, built without a host sync.

    Group g = b * E + e holds the rows of sequence b routed to expert e.  Every group
    starts on a multiple of TILE_ROWS; the tail of its last tile is zero rows.
    Returns (dest [B*N, k] int64, group_offsets [G+1] int32 (padded), group_sizes [G] int32,
    tile_group [T_max] int32 (-1 for unused tiles), rows_padded_max).
    """
    bsz, n, k = expert_idx.shape
    g_count = bsz * num_experts
    dev = expert_idx.device
    gid = (expert_idx.long() + torch.arange(bsz, device=dev)[:, None, None] * num_experts).reshape(-1)
    sizes = torch.bincount(gid, minlength=g_count)
    padded = (sizes + TILE_ROWS - 1) // TILE_ROWS * TILE_ROWS
    ends = torch.cumsum(padded, 0)
    starts = ends - padded
    order = torch.argsort(gid, stable=True)
    sorted_gid = gid[order]
    first = torch.cumsum(sizes, 0) - sizes  # unpadded start of each group in sorted order
    rank_sorted = torch.arange(gid.numel(), device=dev) - first[sorted_gid]
    dest = torch.empty_like(gid)
    dest[order] = starts[sorted_gid] + rank_sorted
    total_rows = bsz * n * k
    t_max = (total_rows + TILE_ROWS - 1) // TILE_ROWS + g_count
    tile_start = torch.arange(t_max, device=dev) * TILE_ROWS
    tile_group = torch.searchsorted(ends, tile_start, right=True)
    tile_group = torch.where(tile_start < ends[-1], tile_group, torch.full_like(tile_group, -1))
    offsets = torch.cat([starts.new_zeros(1), ends]).to(torch.int32)
    return (dest.view(bsz * n, k), offsets, sizes.to(torch.int32), tile_group.to(torch.int32), t_max * TILE_ROWS)


def permute_rows(x: torch.Tensor, dest: torch.Tensor, rows_padded: int) -> torch.Tensor:
    """x: [R, D]; dest: [R, k] -> out [rows_padded, D] with out[dest[i, j]] = x[i]; other rows zero."""
    k = dest.shape[1]
    out = x.new_zeros(rows_padded, x.shape[1])
    src = x if k == 1 else x.repeat_interleave(k, dim=0)
    return out.index_copy(0, dest.reshape(-1), src)


def unpermute_rows(y: torch.Tensor, dest: torch.Tensor, weights: Optional[torch.Tensor]) -> torch.Tensor:
    """y: [rows_padded, D]; out[i] = sum_j weights[i, j] * y[dest[i, j]]."""
    r, k = dest.shape
    g = y.index_select(0, dest.reshape(-1)).view(r, k, -1)
    if weights is not None:
        g = g * weights.unsqueeze(-1).to(g.dtype)
    return g.sum(dim=1)


def _tile_groups(tile_group: torch.Tensor) -> torch.Tensor:
    return tile_group.clamp_min(0).long()


def gg_nt(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor) -> torch.Tensor:
    """out[r] = x[r] @ w[g(r)].T ; x: [R, K], w: [G, N, K] -> [R, N]."""
    t = x.shape[0] // TILE_ROWS
    wt = w.index_select(0, _tile_groups(tile_group)[:t])
    return torch.bmm(x.view(t, TILE_ROWS, -1), wt.transpose(1, 2).to(x.dtype)).view(x.shape[0], -1)


def gg_nn(x: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor) -> torch.Tensor:
    """out[r] = x[r] @ w[g(r)] ; x: [R, K], w: [G, K, N] -> [R, N]."""
    t = x.shape[0] // TILE_ROWS
    wt = w.index_select(0, _tile_groups(tile_group)[:t])
    return torch.bmm(x.view(t, TILE_ROWS, -1), wt.to(x.dtype)).view(x.shape[0], -1)


def gg_tn(a: torch.Tensor, b: torch.Tensor, tile_group: torch.Tensor, num_groups: int,
          out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """out[g] = sum_{r in g} a[r]^T b[r] ; a: [R, M], b: [R, N] -> [G, M, N] (fp32 accumulation)."""
    t = a.shape[0] // TILE_ROWS
    part = torch.bmm(a.view(t, TILE_ROWS, -1).transpose(1, 2), b.view(t, TILE_ROWS, -1)).float()
    # rows of tiles that belong to no group are undefined on the kernel path: select them away (not multiply)
    part = torch.where((tile_group[:t] >= 0).view(-1, 1, 1), part, torch.zeros((), dtype=part.dtype, device=part.device))
    out = torch.zeros(num_groups, a.shape[1], b.shape[1], device=a.device, dtype=torch.float32)
    out.index_add_(0, _tile_groups(tile_group)[:t], part)
    return out.to(out_dtype)


# --------------------------------------------------------------------------- pointwise fast-weight math
def swiglu(y02: torch.Tensor) -> torch.Tensor:
    """y02: [R, 2I] = [gate | up] -> silu(gate) * up."""
    y0, y2 = y02.float().chunk(2, dim=-1)
    return (F.silu(y0) * y2).to(y02.dtype)


def silu_backprop(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    sig = torch.sigmoid(x)
    return dy * sig * (1 + x * (1 - sig))


def fw_write_pointwise(y02: torch.Tensor, dh: torch.Tensor, lr: torch.Tensor):
    """Inner-gradient pointwise block of the fast-weight write.

    y02: [R, 2I] pre-activations (gate | up); dh: [R, I] = (p*v) @ W1; lr: [R, 3] (lr0, lr1, lr2).
    Returns (dy02_lr [R, 2I] = [dgate_pre*lr0 | dup*lr2], h_lr [R, I] = hidden*lr1).
    """
    y0, y2 = y02.float().chunk(2, dim=-1)
    dhf = dh.float()
    lrf = lr.float()
    s = F.silu(y0)
    hidden = s * y2
    dup = dhf * s
    dgate_pre = silu_backprop(dhf * y2, y0)
    dy02 = torch.cat([dgate_pre * lrf[:, 0:1], dup * lrf[:, 2:3]], dim=-1)
    return dy02.to(y02.dtype), (hidden * lrf[:, 1:2]).to(y02.dtype)


# --------------------------------------------------------------------------- Newton-Schulz
NS5_COEFFS = (
    (4.0848, -6.8946, 2.9270),
    (3.9505, -6.3029, 2.6377),
    (3.7418, -5.5913, 2.3037),
    (2.8769, -3.1427, 1.2046),
    (2.8366, -3.0525, 1.2012),
)
NS_FIXED_COEFFS = ((3.4445, -4.7750, 2.0315),) * 5


def newton_schulz(g: torch.Tensor, coeffs=NS5_COEFFS, compute_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Batched Muon orthogonalisation of g: [b, m, n] (iterates on the wide orientation)."""
    assert g.dim() == 3
    dt = compute_dtype or (torch.bfloat16 if g.is_cuda else g.dtype)
    x = g.to(dt)
    tall = g.size(1) > g.size(2)
    if tall:
        x = x.transpose(1, 2)
    x = x / (x.float().norm(dim=(1, 2), keepdim=True) + 1e-7).to(dt)
    for a, b, c in coeffs:
        aa = x @ x.transpose(1, 2)
        bb = b * aa + c * (aa @ aa)
        x = a * x + bb @ x
    if tall:
        x = x.transpose(1, 2)
    return x


# --------------------------------------------------------------------------- loss
def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         chunk: int = 8192) -> Tuple[torch.Tensor, torch.Tensor]:
    """Mean CE over non-ignored labels of (h @ weight.T); logits are formed chunk by chunk.

    h: [T, d], weight: [V, d], labels: [T].  Returns (loss, n_valid).
    """
    total = h.new_zeros((), dtype=torch.float32)
    n_valid = (labels != ignore_index).sum()
    for s in range(0, h.shape[0], chunk):
        logits = (h[s:s + chunk] @ weight.t().to(h.dtype)).float()
        total = total + F.cross_entropy(logits, labels[s:s + chunk], ignore_index=ignore_index, reduction="sum")
    return total / n_valid.clamp_min(1), n_valid


# --------------------------------------------------------------------------- optimizer
def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
               p_lowp: Optional[torch.Tensor] = None) -> None:
    """In-place decoupled-weight-decay Adam on flat fp32 tensors (torch.optim.AdamW semantics)."""
    gf = g.float() * grad_scale
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    p.mul_(1 - lr * weight_decay)
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if p_lowp is not None:
        p_lowp.copy_(p)


# --------------------------------------------------------------------------- NVS
def plucker_rays(fxfycxcy: torch.Tensor, c2w: torch.Tensor, h: int, w: int):
    """Per-pixel camera rays.  fxfycxcy: [b, v, 4] (pixels), c2w: [b, v, 4, 4].

    Returns (ray_o, ray_d): [b, v, 3, h, w] with unit directions
    (uttt_nvs/models/lvsm_moe.py:128-163).
    """
    b, v = fxfycxcy.shape[:2]
    dev = fxfycxcy.device
    y, x = torch.meshgrid(torch.arange(h, device=dev), torch.arange(w, device=dev), indexing="ij")
    x = (x.float() + 0.5)[None, None].expand(b, v, h, w)
    y = (y.float() + 0.5)[None, None].expand(b, v, h, w)
    fx, fy, cx, cy = [fxfycxcy[..., i].float()[..., None, None] for i in range(4)]
    d_cam = torch.stack([(x - cx) / fx, (y - cy) / fy, torch.ones_like(x)], dim=2)  # [b,v,3,h,w]
    rot = c2w[..., :3, :3].float()
    d = torch.einsum("bvij,bvjhw->bvihw", rot, d_cam)
    d = d / d.norm(dim=2, keepdim=True)
    o = c2w[..., :3, 3].float()[..., None, None].expand(b, v, 3, h, w)
    return o, d


def plucker_embed(image: torch.Tensor, fxfycxcy: torch.Tensor, c2w: torch.Tensor, is_target: torch.Tensor,
                  patch: int) -> torch.Tensor:
    """Posed-image tokens before the linear embed.

    image: [b, v, 3, H, W] in [0, 1]; is_target: [v] bool (target views carry zero RGB).
    Channels per pixel: (o, d, o x d, rgb*2-1) = 12; patchified in (ph pw c) order
    -> [b, v, (H/p)*(W/p), p*p*12].  (uttt_nvs/models/lvsm_moe.py:235-258, 183-190)
    """
    b, v, _, hh, ww = image.shape
    o, d = plucker_rays(fxfycxcy, c2w, hh, ww)
    rgb = image.float() * 2.0 - 1.0
    rgb = torch.where(is_target.view(1, v, 1, 1, 1), torch.zeros_like(rgb), rgb)
    x = torch.cat([o, d, torch.cross(o, d, dim=2), rgb], dim=2)  # [b,v,12,H,W]
    c = x.shape[2]
    x = x.view(b, v, c, hh // patch, patch, ww // patch, patch)
    x = x.permute(0, 1, 3, 5, 4, 6, 2).reshape(b, v, (hh // patch) * (ww // patch), patch * patch * c)
    return x
