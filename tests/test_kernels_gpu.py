"""Numerics of every sm_100a kernel against the plain PyTorch fp32 statement of the same op."""
import math
import os

import pytest
import torch
import torch.nn.functional as F

from uttt_b200 import ops
from uttt_b200.ops import reference as ref
from uttt_b200.ops import functional as fn
from uttt_b200.ops._ext import load

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ext():
    ext = load(required=True)
    return ext


def _close(a, b, atol, rtol, msg=""):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol, msg=lambda m: f"{msg}: {m}")


def _status_ok():
    st = _ext().gemm_status(torch.zeros(1, device=DEV))
    assert int(st[0].item()) == 0, f"a tensor-core kernel reported a timed-out wait (code {int(st[0])})"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [384, 1536])
def test_rms_norm(dtype, d):
    _ext()
    torch.manual_seed(0)
    x = torch.randn(777, d, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(d, device=DEV, dtype=dtype) * 0.1 + 1).requires_grad_(True)
    y = ops.rms_norm(x, w, 1e-6)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = ref.rms_norm(xr, wr, 1e-6)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(y, yr, tol, tol)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    _close(x.grad, xr.grad, tol, tol, "dx")
    _close(w.grad, wr.grad, 0.5 if dtype == torch.bfloat16 else 1e-3, 3e-2 if dtype == torch.bfloat16 else 1e-4, "dw")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [384, 1536])
def test_add_rms_norm(dtype, d):
    """Residual addition fused with the norm: both outputs and all three gradients against fp32 PyTorch."""
    _ext()
    torch.manual_seed(1)
    x = torch.randn(515, d, device=DEV, dtype=dtype, requires_grad=True)
    delta = torch.randn(515, d, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(d, device=DEV, dtype=dtype) * 0.1 + 1).requires_grad_(True)
    s, y = ops.add_rms_norm(x, delta, w, 1e-6)
    gs, gy = torch.randn_like(s), torch.randn_like(y)
    (s.float() * gs.float()).sum().add((y.float() * gy.float()).sum()).backward()
    xr, dr, wr = (t.detach().float().requires_grad_(True) for t in (x, delta, w))
    sr = (xr + dr).to(dtype).float() if dtype == torch.bfloat16 else xr + dr
    sr_live = xr + dr
    yr = ref.rms_norm(sr_live, wr, 1e-6)
    ((sr_live * gs.float()).sum() + (yr * gy.float()).sum()).backward()
    tol = dict(atol=3e-2, rtol=3e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    _close(s, sr, 1e-6 if dtype == torch.float32 else 0.0, 0.0, "sum")       # the rounded sum itself is exact
    _close(y, yr, **tol, msg="y")
    _close(x.grad, xr.grad, **tol, msg="dx")
    _close(delta.grad, dr.grad, **tol, msg="ddelta")
    wtol = dict(atol=0.5, rtol=5e-2) if dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-4)
    _close(w.grad, wr.grad, **wtol, msg="dw")
    # only the norm output used downstream: the gradient of the sum is absent
    x2 = x.detach().clone().requires_grad_(True)
    _, y2 = ops.add_rms_norm(x2, delta.detach(), w.detach(), 1e-6)
    y2.float().mul(gy.float()).sum().backward()
    xr2 = x.detach().float().requires_grad_(True)
    ref.rms_norm(xr2 + delta.detach().float(), w.detach().float(), 1e-6).mul(gy.float()).sum().backward()
    _close(x2.grad, xr2.grad, **tol, msg="dx (norm output only)")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_gather_and_scatter_add(dtype):
    """Embedding lookup and its table gradient (fp32 vector reductions) against torch, with a skewed id
    distribution, a padding row and an out-of-range id (skipped, status 73, no fault)."""
    ext = _ext()
    torch.manual_seed(2)
    vocab, d = 1000, 384
    table = torch.randn(vocab, d, device=DEV, dtype=dtype, requires_grad=True)
    ids = (torch.rand(4, 2048, device=DEV) ** 4 * vocab).long().clamp_(0, vocab - 1)      # many repeats of low ids
    ids[0, :7] = 5                                                                        # padding rows
    out = ops.embedding(ids, table, padding_idx=5)
    assert torch.equal(out, table.detach()[ids])
    gy = torch.randn_like(out)
    out.backward(gy)
    tr = table.detach().float().requires_grad_(True)
    F.embedding(ids, tr, padding_idx=5).backward(gy.float())
    tol = dict(atol=0.25, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-4)
    _close(table.grad, tr.grad, **tol, msg="dtable")
    assert float(table.grad[5].abs().max()) == 0.0
    _status_ok()
    bad = ids.clone()
    bad[1, 3] = vocab + 17
    o2 = ext.embedding_fwd(table.detach(), bad)
    assert float(o2[1, 3].abs().max()) == 0.0 and torch.equal(o2[0], out[0])
    st = ext.gemm_status(torch.zeros(1, device=DEV))
    assert int(st[0].item()) == 73
    st.zero_()


@pytest.mark.parametrize("hd", [64, 96])
def test_rope(hd):
    _ext()
    x = torch.randn(2, 300, 5, hd, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.rope(x, 1000, 1e6)
    yr = ref.rope(x.detach().float(), 1000, 1e6)
    _close(y, yr, 2e-2, 2e-2)
    g = torch.randn_like(y)
    (gx,) = torch.autograd.grad(y, x, g)
    _close(gx, ref.rope(g.float(), 1000, 1e6, inverse=True), 2e-2, 2e-2)


@pytest.mark.parametrize("norm", ["l2", "rms", None])
@pytest.mark.parametrize("heads,D,rope_dim", [(4, 96, 32),      # warp form, 6 vector pairs per head
                                              (4, 384, 96),     # warp form, the 760M shape (24 pairs, 96-wide sub-heads)
                                              (2, 768, 256),    # warp form, two pairs per lane
                                              (3, 72, 24)])     # block form (odd number of vectors per head)
def test_fw_qk_prep(norm, heads, D, rope_dim):
    _ext()
    torch.manual_seed(1)
    b, l = 2, 160
    d = heads * D
    x = torch.randn(b, l, d, device=DEV, dtype=torch.float32, requires_grad=True)
    sc = (torch.randn(d, device=DEV) * 0.1 + 1).requires_grad_(True)
    sh = (torch.randn(d, device=DEV) * 0.1).requires_grad_(True)
    y = ops.fw_qk_prep(x, sc, sh, heads, rope_dim, 1e6, 64, True, norm)
    xr, scr, shr = [t.detach().clone().requires_grad_(True) for t in (x, sc, sh)]
    yr = ref.fw_qk_prep(xr, scr, shr, heads, rope_dim, 1e6, 64, True, norm)
    _close(y, yr, 1e-4, 1e-4)
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g)
    _close(x.grad, xr.grad, 1e-4, 1e-3, "dx")
    _close(sc.grad, scr.grad, 2e-3, 1e-3, "dscale")
    _close(sh.grad, shr.grad, 2e-3, 1e-3, "dshift")
    # bf16 path
    xb = x.detach().bfloat16()
    yb = ops.fw_qk_prep(xb, sc.detach().bfloat16(), sh.detach().bfloat16(), heads, rope_dim, 1e6, 64, True, norm)
    _close(yb, yr, 3e-2, 3e-2)


def test_swiglu_and_second_order():
    _ext()
    torch.manual_seed(2)
    y02 = torch.randn(257, 2 * 192, device=DEV, requires_grad=True)
    h = ops.swiglu(y02)
    yr = y02.detach().clone().requires_grad_(True)
    hr = ref.swiglu(yr)
    _close(h, hr, 1e-5, 1e-5)
    dh = torch.randn_like(h, requires_grad=True)
    dhr = dh.detach().clone().requires_grad_(True)
    (g1,) = torch.autograd.grad(h, y02, dh, create_graph=True)
    (g1r,) = torch.autograd.grad(hr, yr, dhr, create_graph=True)
    _close(g1, g1r, 1e-5, 1e-4)
    c = torch.randn_like(g1)
    gg = torch.autograd.grad(g1, [dh, y02], c)
    ggr = torch.autograd.grad(g1r, [dhr, yr], c)
    for a, b_ in zip(gg, ggr):
        _close(a, b_, 1e-4, 1e-3)


def test_fw_write_pointwise():
    _ext()
    torch.manual_seed(3)
    r, inter = 300, 128
    y02 = torch.randn(r, 2 * inter, device=DEV, requires_grad=True)
    dh = torch.randn(r, inter, device=DEV, requires_grad=True)
    lr = (torch.rand(r, 3, device=DEV) * 0.1).requires_grad_(True)
    a, b_ = ops.fw_write_pointwise(y02, dh, lr)
    ins_r = [t.detach().clone().requires_grad_(True) for t in (y02, dh, lr)]
    ar, br = ref.fw_write_pointwise(*ins_r)
    _close(a, ar, 1e-5, 1e-4)
    _close(b_, br, 1e-5, 1e-4)
    ca, cb = torch.randn_like(a), torch.randn_like(b_)
    got = torch.autograd.grad([a, b_], [y02, dh, lr], [ca, cb])
    want = torch.autograd.grad([ar, br], ins_r, [ca, cb])
    for x, y in zip(got, want):
        _close(x, y, 1e-4, 1e-3)


def _plan(bsz=2, n=700, e=4, k=2, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    logits = torch.randn(bsz, n, e, generator=g)
    idx = logits.topk(k, -1).indices.to(DEV)
    return ops.build_group_plan(idx, e)


@pytest.mark.parametrize("bsz,n,e,k", [(2, 700, 4, 2), (3, 5000, 32, 2), (1, 64, 1, 1), (2, 2048, 96, 1),
                                       # small exhaustive shapes: empty groups, groups of one row, odd expert counts
                                       (1, 3, 5, 2), (2, 1, 3, 1), (4, 129, 2, 2), (1, 128, 5, 1), (3, 2, 2, 2)])
def test_group_plan_kernel_matches_reference(bsz, n, e, k):
    _ext()
    g = torch.Generator().manual_seed(n)
    idx = torch.randn(bsz, n, e, generator=g).topk(k, -1).indices.to(DEV)
    plan = ops.build_group_plan(idx, e)
    dest, offsets, sizes, tile_group, rows = ref.build_group_plan(idx, e)
    assert plan.rows_padded == rows
    assert torch.equal(plan.sizes.cpu(), sizes.cpu()) and torch.equal(plan.offsets.cpu(), offsets.cpu())
    assert torch.equal(plan.tile_group.cpu(), tile_group.cpu())
    assert torch.equal(plan.dest.cpu(), dest.cpu())          # same stable (token-major) order inside groups


@pytest.mark.parametrize("d,e,k,renorm,bias_in_logits,dtype", [(384, 32, 2, False, False, torch.bfloat16),
                                                               (192, 64, 4, True, False, torch.bfloat16),
                                                               (128, 8, 1, False, True, torch.float32),
                                                               (512, 16, 2, True, False, torch.bfloat16)])
def test_fused_router_matches_reference(d, e, k, renorm, bias_in_logits, dtype):
    _ext()
    torch.manual_seed(21)
    bsz, n = 3, 1003
    rows = torch.randn(bsz, n, d, device=DEV).to(dtype).requires_grad_(True)
    router = (torch.randn(e, d, device=DEV) * 0.2).requires_grad_(True)
    bias = torch.randn(e, device=DEV) * 0.05
    idx, w, psum = ops.route_softmax_topk(rows, router, bias, k, 0.7, bias_in_logits, renorm)
    rr = rows.detach().float().requires_grad_(True)
    rt = router.detach().clone().requires_grad_(True)
    logits = rr @ rt.t()
    if bias_in_logits:
        logits = logits + bias
    probs = torch.softmax(logits, -1)
    scores = logits.detach() if bias_in_logits else logits.detach() + bias
    # selection must agree wherever the k-th and (k+1)-th scores are not nearly tied
    top = torch.topk(scores, k + 1 if k < e else k, dim=-1)
    clear = (top.values[..., k - 1] - top.values[..., -1]).abs() > 1e-3 if k < e else torch.ones_like(idx[..., 0]).bool()
    want_idx = top.indices[..., :k]
    assert bool((idx.long().sort(-1).values == want_idx.sort(-1).values)[clear].all())
    picked = probs.gather(-1, idx.long())
    if renorm:
        picked = picked / picked.sum(-1, keepdim=True).clamp_min(1e-9)
    wr = (picked * 0.7).view(bsz * n, k)
    _close(w, wr, 1e-4, 1e-3, "weights")
    _close(psum, probs.sum(1), 1e-2, 1e-3, "probs_sum")
    gw = torch.randn_like(w)
    gp = torch.randn_like(psum) * 0.1
    g1, g2 = torch.autograd.grad([w, psum], [rows, router], [gw, gp])
    g1r, g2r = torch.autograd.grad([wr, probs.sum(1)], [rr, rt], [gw, gp])
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    _close(g1, g1r, tol, tol, "drows")
    _close(g2, g2r, 2e-3, 2e-3, "drouter")


@pytest.mark.parametrize("router_type,scale", [("norm_softmax", 0.0), ("norm_relu", 0.0), ("norm_relu", 3.0)])
@pytest.mark.parametrize("d,e,k,renorm,dtype", [(384, 32, 2, False, torch.bfloat16), (192, 64, 4, True, torch.float32)])
def test_fused_router_normalised_modes(router_type, scale, d, e, k, renorm, dtype):
    """The L2-normalised router variants (scores = scale * logits / |logits|, softmax or rectified) in the fused
    kernel: selection, weights, probability sums and both gradients against the fp32 PyTorch statement."""
    _ext()
    torch.manual_seed(22)
    bsz, n = 2, 777
    rows = torch.randn(bsz, n, d, device=DEV).to(dtype).requires_grad_(True)
    router = (torch.randn(e, d, device=DEV) * 0.2).requires_grad_(True)
    bias = torch.randn(e, device=DEV) * 0.02
    idx, w, psum = ops.route_topk(rows, router, bias, k, 0.7, False, renorm, router_type, scale, 1e-6)
    rr = rows.detach().float().requires_grad_(True)
    rt = router.detach().clone().requires_grad_(True)
    sel, probs = ref.route_scores(rr @ rt.t(), router_type, scale, 1e-6)
    scores = sel.detach() + bias
    top = torch.topk(scores, k + 1, dim=-1)
    clear = (top.values[..., k - 1] - top.values[..., -1]).abs() > 1e-3
    assert bool((idx.long().sort(-1).values == top.indices[..., :k].sort(-1).values)[clear].all())
    picked = probs.gather(-1, idx.long())
    if renorm:
        picked = picked / picked.sum(-1, keepdim=True).clamp_min(1e-9)
    wr = (picked * 0.7).view(bsz * n, k)
    _close(w, wr, 1e-4, 1e-3, "weights")
    _close(psum, probs.sum(1), 1e-2, 1e-3, "probs_sum")
    gw = torch.randn_like(w)
    gp = torch.randn_like(psum) * 0.1
    g1, g2 = torch.autograd.grad([w, psum], [rows, router], [gw, gp])
    g1r, g2r = torch.autograd.grad([wr, probs.sum(1)], [rr, rt], [gw, gp])
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-4
    _close(g1, g1r, tol, tol, "drows")
    _close(g2, g2r, 3e-3, 3e-3, "drouter")


@pytest.mark.parametrize("renorm", ["restore", "unit", "none"])
@pytest.mark.parametrize("d,ddtype", [(384, torch.bfloat16), (1536, torch.float32), (200, torch.bfloat16)])
def test_pool_step_matches_reference(renorm, d, ddtype):
    _ext()
    torch.manual_seed(22)
    m = torch.randn(3, 5, 70, d, device=DEV, requires_grad=True)
    dd = torch.randn(3, 5, 70, d, device=DEV).to(ddtype).requires_grad_(True)
    n, w = ops.pool_step(m, dd, 0.3, renorm)
    assert w.dtype == torch.bfloat16 and n.dtype == torch.float32
    mr = m.detach().clone().requires_grad_(True)
    dr = dd.detach().float().requires_grad_(True)
    u = mr + dr * 0.3
    if renorm == "restore":
        nr = u / (u.norm(dim=-1, keepdim=True) + 1e-5) * mr.norm(dim=-1, keepdim=True)
    elif renorm == "unit":
        nr = F.normalize(u, dim=-1)
    else:
        nr = u
    _close(n, nr, 1e-5, 1e-5, "n")
    _close(w, nr, 2e-2, 1e-2, "w")
    gn = torch.randn_like(n)
    gw = torch.randn_like(n).bfloat16()
    g1, g2 = torch.autograd.grad([n, w], [m, dd], [gn, gw], retain_graph=True)
    g1r, g2r = torch.autograd.grad(nr, [mr, dr], gn + gw.float(), retain_graph=True)
    _close(g1, g1r, 1e-4, 1e-4, "dm")
    _close(g2, g2r, 3e-2 if ddtype == torch.bfloat16 else 1e-4, 1e-2 if ddtype == torch.bfloat16 else 1e-4, "dd")
    (g3,) = torch.autograd.grad(w, m, gw)            # only the compute copy has a gradient
    (g3r,) = torch.autograd.grad(nr, mr, gw.float())
    _close(g3, g3r, 1e-4, 1e-4, "dm from w")


def test_permute_unpermute():
    _ext()
    plan = _plan()
    r, k = plan.dest.shape
    x = torch.randn(r, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    xp = ops.permute_rows(x, plan)
    xpr = ref.permute_rows(x.detach().float(), plan.dest, plan.rows_padded)
    # rows of groups (their zero padding included) are defined; tiles past the last group are never read
    live = int(plan.offsets[-1])
    _close(xp[:live], xpr[:live], 0, 0)
    w = torch.rand(r, k, device=DEV, requires_grad=True)
    yp = torch.randn(plan.rows_padded, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = ops.unpermute_rows(yp, plan, w)
    ypr = yp.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    outr = ref.unpermute_rows(ypr, plan.dest, wr)
    _close(out, outr, 2e-2, 2e-2)
    g = torch.randn_like(out)
    gy, gw = torch.autograd.grad(out, [yp, w], g)
    gyr, gwr = torch.autograd.grad(outr, [ypr, wr], g.float())
    _close(gy[:live], gyr[:live], 2e-2, 2e-2)
    _close(gw, gwr, 0.15, 3e-2)
    (gx,) = torch.autograd.grad(xp, x, torch.ones_like(xp))
    _close(gx, torch.full_like(gx, float(k)), 0, 0)
    # weighted scatter (value rows scaled by their combine weight) and its gradients
    w2 = torch.rand(r, k, device=DEV, requires_grad=True)
    xs = ops.permute_rows(x, plan, w2)
    xr = x.detach().float().requires_grad_(True)
    w2r = w2.detach().clone().requires_grad_(True)
    scaled = (xr.unsqueeze(1) * w2r.unsqueeze(-1)).reshape(-1, 128)
    xsr = torch.zeros(plan.rows_padded, 128, device=DEV).index_copy(0, plan.dest.reshape(-1), scaled)
    _close(xs[:live], xsr[:live], 2e-2, 2e-2)
    c = torch.randn_like(xs)
    ga, gb = torch.autograd.grad(xs, [x, w2], c)
    gar, gbr = torch.autograd.grad(xsr, [xr, w2r], c.float())
    _close(ga, gar, 3e-2, 3e-2)
    _close(gb, gbr, 0.2, 3e-2)


@pytest.mark.parametrize("k,n", [(128, 256), (384, 3072), (64, 64), (1536, 384), (128, 128)])
def test_gg_nt(k, n):
    _ext()
    torch.manual_seed(4)
    plan = _plan(seed=k)
    g = plan.num_groups
    x = torch.randn(plan.rows_padded, k, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(g, n, k, device=DEV) / math.sqrt(k)).bfloat16()
    out = ops.gg_nt(x, w, plan)
    want = ref.gg_nt(x.float(), w.float(), plan.tile_group)
    torch.cuda.synchronize()
    _status_ok()
    # unused tiles are defined as zero by the kernel; the reference multiplies them by group 0
    used = (plan.tile_group >= 0).repeat_interleave(128)
    _close(out[used], want[used], 3e-2, 3e-2)
    assert float(out[~used].abs().max() if (~used).any() else 0) == 0.0


@pytest.mark.parametrize("k,n", [(128, 256), (384, 1536), (64, 64), (128, 384)])
def test_gg_nn(k, n):
    _ext()
    torch.manual_seed(5)
    plan = _plan(seed=k + 1)
    g = plan.num_groups
    x = torch.randn(plan.rows_padded, k, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(g, k, n, device=DEV) / math.sqrt(k)).bfloat16()
    out = ops.gg_nn(x, w, plan)
    want = ref.gg_nn(x.float(), w.float(), plan.tile_group)
    torch.cuda.synchronize()
    _status_ok()
    used = (plan.tile_group >= 0).repeat_interleave(128)
    _close(out[used], want[used], 3e-2, 3e-2)


@pytest.mark.parametrize("m,n", [(128, 128), (384, 192), (256, 64), (256, 384), (128, 512), (64, 128), (64, 64)])
def test_gg_tn(m, n):
    _ext()
    torch.manual_seed(6)
    plan = _plan(seed=m)
    used = (plan.tile_group >= 0).repeat_interleave(128).unsqueeze(1)
    a = torch.randn(plan.rows_padded, m, device=DEV, dtype=torch.bfloat16) * used
    b_ = torch.randn(plan.rows_padded, n, device=DEV, dtype=torch.bfloat16) * used
    # zero the padding rows of every group (the layout contract)
    real = torch.zeros(plan.rows_padded, 1, device=DEV, dtype=torch.bool)
    real[plan.dest.reshape(-1)] = True
    a = a * real
    b_ = b_ * real
    # rows of tiles past the last group are undefined by contract: make them NaN to prove nobody reads them
    live = int(plan.offsets[-1])
    a[live:] = float("nan")
    b_[live:] = float("nan")
    out = ops.gg_tn(a, b_, plan)
    want = ref.gg_tn(a.float(), b_.float(), plan.tile_group, plan.num_groups)
    torch.cuda.synchronize()
    _status_ok()
    _close(out, want, 0.3, 2e-2)
    if m % 128 != 0:
        return
    # fp32 output accumulated in place over two launches (the memory-side reduce-add epilogue)
    from uttt_b200.ops._ext import load
    acc = torch.full((plan.num_groups, m, n), 0.25, device=DEV)
    for _ in range(2):
        load().gg_tn_segments(a, b_, plan.offsets, plan.num_groups, 1, torch.float32, acc)
    torch.cuda.synchronize()
    _status_ok()
    _close(acc, 0.25 + 2 * want, 0.3, 2e-2)


def _rel_fro(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


@pytest.mark.parametrize("k,inter", [(128, 128), (384, 1536), (64, 256)])
def test_gg_swiglu_fused_epilogue(k, inter):
    """SwiGLU applied in the grouped GEMM's epilogue = silu(x W0^T) * (x W2^T) in fp32, forward and gradients."""
    _ext()
    torch.manual_seed(14)
    plan = _plan(seed=k + inter)
    g = plan.num_groups
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    used = (plan.tile_group >= 0).repeat_interleave(128)
    x = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16().requires_grad_(True)
    w = (torch.randn(g, 2 * inter, k, device=DEV) / math.sqrt(k)).bfloat16().requires_grad_(True)
    hid = ops.gg_swiglu(x, w, plan)
    assert hid.shape == (plan.rows_padded, inter)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    y = ref.gg_nt(xr, wr, plan.tile_group)
    want = F.silu(y[:, :inter]) * y[:, inter:]
    torch.cuda.synchronize()
    _status_ok()
    _close(hid[used], want[used], 3e-2, 3e-2, "hidden")
    assert _rel_fro(hid[used], want[used]) < 1e-2
    assert float(hid[~used].abs().max() if (~used).any() else 0) == 0.0
    c = torch.randn_like(hid) * real.bfloat16()
    gx, gw = torch.autograd.grad(hid, [x, w], c)
    gxr, gwr = torch.autograd.grad(want, [xr, wr], c.float())
    torch.cuda.synchronize()
    _status_ok()
    _close(gx[used], gxr[used], 8e-2, 3e-2, "dx")
    assert _rel_fro(gx[used], gxr[used]) < 1.5e-2
    _close(gw, gwr, 0.5, 3e-2, "dw")
    assert _rel_fro(gw, gwr) < 1.5e-2


@pytest.mark.parametrize("with_lr,want_y", [(True, False), (True, True), (False, False)])
def test_gg_swiglu_write_epilogue(with_lr, want_y):
    """The write's point-wise block in the GEMM epilogue: dy02 * lr, hidden * lr1 and (optionally) y02."""
    ext = _ext()
    torch.manual_seed(15)
    k, inter = 128, 256
    plan = _plan(seed=77)
    g = plan.num_groups
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    used = (plan.tile_group >= 0).repeat_interleave(128)
    x = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16()
    w = (torch.randn(g, 2 * inter, k, device=DEV) / math.sqrt(k)).bfloat16()
    dh = (torch.randn(plan.rows_padded, inter, device=DEV) * real).bfloat16()
    lr = (torch.rand(plan.rows_padded, 3, device=DEV) + 0.5) if with_lr else None
    dy02, hlr, y02 = ext.gg_nt_swiglu_bwd(x, w, dh, lr, plan.tile_group, True, want_y)
    torch.cuda.synchronize()
    _status_ok()
    y = ref.gg_nt(x.float(), w.float(), plan.tile_group)
    y0, y2, d = y[:, :inter], y[:, inter:], dh.float()
    sg = torch.sigmoid(y0)
    l = lr if with_lr else torch.ones(plan.rows_padded, 3, device=DEV)
    want_g = d * y2 * (sg * (1 + y0 * (1 - sg))) * l[:, 0:1]
    want_u = d * F.silu(y0) * l[:, 2:3]
    want_h = F.silu(y0) * y2 * l[:, 1:2]
    for name, got, want in (("dy0", dy02[:, :inter], want_g), ("dy2", dy02[:, inter:], want_u), ("hlr", hlr, want_h)):
        _close(got[used], want[used], 4e-2, 3e-2, name)
        assert _rel_fro(got[used], want[used]) < 1e-2, name
        assert float(got[~used].abs().max() if (~used).any() else 0) == 0.0
    if want_y:
        _close(y02[used], y[used], 3e-2, 2e-2, "y02")
    # same numbers as the unfused sequence within bf16 rounding of the intermediate
    y02_ref = ops.gg_nt(x, w, plan)
    a, b_ = ext.fw_write_pw_fwd(y02_ref, dh, l.contiguous())
    assert _rel_fro(dy02[used], a[used]) < 1.5e-2 and _rel_fro(hlr[used], b_[used]) < 1.5e-2


def test_fw_write_grad_uses_fused_epilogue_and_matches_reference():
    """Inner gradient of the write and its gradient-of-gradient through the fused kernels vs fp32 autograd."""
    _ext()
    torch.manual_seed(16)
    k, inter = 128, 128
    plan = _plan(bsz=2, n=300, e=4, k=2, seed=5)
    g = plan.num_groups
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    kp = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16().requires_grad_(True)
    vp = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16().requires_grad_(True)
    lrp = ((torch.rand(plan.rows_padded, 3, device=DEV) * 0.5 + 0.5) * real).requires_grad_(True)
    w02 = (torch.randn(g, 2 * inter, k, device=DEV) / math.sqrt(k)).bfloat16().requires_grad_(True)
    w1 = (torch.randn(g, k, inter, device=DEV) / math.sqrt(inter)).bfloat16().requires_grad_(True)
    g02, g1 = ops.fw_write_grad(kp, vp, lrp, w02, w1, plan)
    c02, c1 = torch.randn_like(g02) * 0.1, torch.randn_like(g1) * 0.1
    grads = torch.autograd.grad([g02, g1], [kp, vp, lrp, w02, w1], [c02, c1])
    f = [t.detach().float().requires_grad_(True) for t in (kp, vp, lrp, w02, w1)]
    y = ref.gg_nt(f[0], f[3], plan.tile_group)
    dhr = ref.gg_nn(f[1], f[4], plan.tile_group)
    a, b_ = ref.fw_write_pointwise(y, dhr, f[2])
    g02r = ref.gg_tn(a, f[0], plan.tile_group, g)
    g1r = ref.gg_tn(f[1], b_, plan.tile_group, g)
    gradsr = torch.autograd.grad([g02r, g1r], f, [c02.float(), c1.float()])
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_fro(g02, g02r) < 1.5e-2 and _rel_fro(g1, g1r) < 1.5e-2
    for name, got, want in zip(("d_kp", "d_vp", "d_lr", "d_w02", "d_w1"), grads, gradsr):
        assert _rel_fro(got, want) < 3e-2, (name, _rel_fro(got, want))


def _pair_plan_reference(tile_group, offsets, tiles):
    out = []
    tg = tile_group.tolist()
    off = offsets.tolist()
    for t in range(tiles):
        g = tg[t]
        if g < 0:
            out.append((-t - 2, -1))
        elif (t - off[g] // 128) % 2 == 0:
            out.append((t, t + 1 if t + 1 < tiles and tg[t + 1] == g else -1))
    return out


@pytest.mark.parametrize("bsz,n,e,k", [(2, 700, 4, 2), (3, 5000, 32, 2), (1, 3, 5, 2), (4, 129, 2, 2), (2, 2048, 96, 1)])
def test_pair_plan(bsz, n, e, k):
    ext = _ext()
    plan = _plan(bsz, n, e, k, seed=n)
    tiles = plan.rows_padded // 128
    entries, count = ext.pair_plan(plan.tile_group, plan.offsets, tiles)
    want = _pair_plan_reference(plan.tile_group.cpu(), plan.offsets.cpu(), tiles)
    assert int(count[0]) == len(want)
    assert entries[:len(want)].cpu().tolist() == [list(w) for w in want]


@pytest.fixture
def one_cta_then_pairs():
    """Yields a function that runs ``f`` with the one-CTA kernels and then with CTA pairs."""
    def run(f):
        try:
            fn.set_cta_pairs(False)
            a = f()
            fn.set_cta_pairs(True)
            b_ = f()
        finally:
            fn.set_cta_pairs(True)
        return a, b_
    return run


@pytest.mark.parametrize("mode,k,n", [("nt", 384, 3072), ("nt", 1536, 384), ("nt", 64, 128), ("nt", 128, 256),
                                      ("nn", 384, 1536), ("nn", 3072, 384), ("nn", 64, 128), ("nn", 128, 640)])
def test_gg_pair_kernels(mode, k, n, one_cta_then_pairs):
    """Two-CTA (cta_group::2) NT / NN products: equal to the one-CTA kernels and to fp32, unused tiles zero."""
    _ext()
    torch.manual_seed(21)
    # 3 experts x 2 sequences with ~230 routed rows each: groups of one and two tiles, odd and even counts
    plan = _plan(bsz=2, n=350, e=3, k=2, seed=k + n)
    g = plan.num_groups
    x = torch.randn(plan.rows_padded, k, device=DEV, dtype=torch.bfloat16)
    shape = (g, n, k) if mode == "nt" else (g, k, n)
    w = (torch.randn(*shape, device=DEV) / math.sqrt(k)).bfloat16()
    op = ops.gg_nt if mode == "nt" else ops.gg_nn
    one, two = one_cta_then_pairs(lambda: op(x, w, plan))
    torch.cuda.synchronize()
    _status_ok()
    want = (ref.gg_nt if mode == "nt" else ref.gg_nn)(x.float(), w.float(), plan.tile_group)
    used = (plan.tile_group >= 0).repeat_interleave(128)
    _close(two[used], want[used], 3e-2, 3e-2, "pairs vs fp32")
    assert _rel_fro(two[used], want[used]) < 1e-2
    _close(two[used], one[used], 1e-2, 1e-2, "pairs vs one CTA")
    assert float(two[~used].abs().max() if (~used).any() else 0) == 0.0


def test_gg_pair_fused_epilogues(one_cta_then_pairs):
    ext = _ext()
    torch.manual_seed(22)
    k, inter = 384, 256
    plan = _plan(bsz=2, n=350, e=3, k=2, seed=9)
    g = plan.num_groups
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    used = (plan.tile_group >= 0).repeat_interleave(128)
    x = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16()
    w = (torch.randn(g, 2 * inter, k, device=DEV) / math.sqrt(k)).bfloat16()
    dh = (torch.randn(plan.rows_padded, inter, device=DEV) * real).bfloat16()
    lr = torch.rand(plan.rows_padded, 3, device=DEV) + 0.5
    one, two = one_cta_then_pairs(lambda: ops.gg_swiglu(x, w, plan))
    y = ref.gg_nt(x.float(), w.float(), plan.tile_group)
    want = F.silu(y[:, :inter]) * y[:, inter:]
    torch.cuda.synchronize()
    _status_ok()
    assert _rel_fro(two[used], want[used]) < 1e-2 and _rel_fro(two[used], one[used]) < 1e-3
    assert float(two[~used].abs().max() if (~used).any() else 0) == 0.0
    one, two = one_cta_then_pairs(lambda: fn._swiglu_bwd_kernel(x, w, dh, lr, plan, True, True))
    torch.cuda.synchronize()
    _status_ok()
    for a, b_ in zip(one, two):
        assert _rel_fro(b_[used], a[used]) < 1e-3
        assert float(b_[~used].abs().max() if (~used).any() else 0) == 0.0


def test_gg_tn_multi_reduces_several_layouts_in_one_launch():
    """Three row buffers with three different routings reduced into one fp32 accumulator in one launch equal the
    sum of the three separate reductions (and the stash that the aggregate write uses gives the same sums)."""
    ext = _ext()
    torch.manual_seed(23)
    m, n = 256, 384
    plans = [_plan(bsz=2, n=300 + 40 * i, e=3, k=2, seed=50 + i) for i in range(3)]
    g = plans[0].num_groups
    a_s, b_s, want = [], [], torch.zeros(g, m, n, device=DEV)
    for plan in plans:
        real = torch.zeros(plan.rows_padded, 1, device=DEV, dtype=torch.bool)
        real[plan.dest.reshape(-1)] = True
        a = (torch.randn(plan.rows_padded, m, device=DEV) * real).bfloat16()
        b_ = (torch.randn(plan.rows_padded, n, device=DEV) * real).bfloat16()
        live = int(plan.offsets[-1])
        a[live:] = float("nan")                 # rows past the last group are never read
        b_[live:] = float("nan")
        a_s.append(a)
        b_s.append(b_)
        want += ref.gg_tn(a.float().nan_to_num(), b_.float().nan_to_num(), plan.tile_group, g)
    acc = torch.full((g, m, n), 0.5, device=DEV)
    ext.gg_tn_multi(a_s, b_s, [p.offsets for p in plans], g, torch.float32, acc)
    torch.cuda.synchronize()
    _status_ok()
    _close(acc, 0.5 + want, 0.3, 2e-2)
    assert _rel_fro(acc - 0.5, want) < 1e-2
    one = ext.gg_tn_multi(a_s[:1], b_s[:1], [plans[0].offsets], g, torch.float32, None)
    _close(one, ref.gg_tn(a_s[0].float().nan_to_num(), b_s[0].float().nan_to_num(), plans[0].tile_group, g), 0.3, 2e-2)


def test_write_stash_matches_per_layer_accumulation():
    _ext()
    torch.manual_seed(24)
    k, inter = 128, 128
    layers = 5                                   # more than one stash-full
    g = None
    runs = {}
    for use_stash in (False, True):
        torch.manual_seed(24)
        acc02 = acc1 = None
        stash = None
        for l in range(layers):
            plan = _plan(bsz=2, n=300, e=4, k=2, seed=70 + l)
            g = plan.num_groups
            real = torch.zeros(plan.rows_padded, 1, device=DEV)
            real[plan.dest.reshape(-1)] = 1
            kp = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16()
            vp = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16()
            lrp = (torch.rand(plan.rows_padded, 3, device=DEV) * 0.5 + 0.5) * real
            if l == 0:
                w02 = (torch.randn(g, 2 * inter, k, device=DEV) / math.sqrt(k)).bfloat16()
                w1 = (torch.randn(g, k, inter, device=DEV) / math.sqrt(inter)).bfloat16()
                acc02 = torch.zeros(g, 2 * inter, k, device=DEV)
                acc1 = torch.zeros(g, k, inter, device=DEV)
                stash = ops.write_stash_for(acc02) if use_stash else None
                assert (stash is not None) == use_stash
            acc02, acc1 = ops.fw_write_grad_accumulate(kp, vp, lrp, w02, w1, plan, acc02, acc1, stash, l == layers - 1)
        torch.cuda.synchronize()
        assert stash is None or stash.pending == 0
        runs[use_stash] = (acc02.clone(), acc1.clone())
    _status_ok()
    assert _rel_fro(runs[True][0], runs[False][0]) < 1e-5 and _rel_fro(runs[True][1], runs[False][1]) < 1e-5


def test_gg_autograd_matches_reference():
    _ext()
    torch.manual_seed(7)
    plan = _plan(seed=11)
    g, k, n = plan.num_groups, 128, 256
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    x = (torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16().requires_grad_(True)
    w = (torch.randn(g, n, k, device=DEV) / math.sqrt(k)).bfloat16().requires_grad_(True)
    out = ops.gg_nt(x, w, plan)
    c = (torch.randn_like(out) * real.bfloat16())
    gx, gw = torch.autograd.grad(out, [x, w], c)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    outr = ref.gg_nt(xr, wr, plan.tile_group)
    gxr, gwr = torch.autograd.grad(outr, [xr, wr], c.float())
    used = (plan.tile_group >= 0).repeat_interleave(128)
    _close(gx[used], gxr[used], 5e-2, 3e-2)
    _close(gw, gwr, 0.5, 3e-2)
    _status_ok()


def test_bmm_nt_and_newton_schulz():
    _ext()
    torch.manual_seed(8)
    a = torch.randn(6, 128, 256, device=DEV, dtype=torch.bfloat16)
    b_ = torch.randn(6, 192, 256, device=DEV, dtype=torch.bfloat16)
    d = torch.randn(6, 128, 192, device=DEV, dtype=torch.bfloat16)
    out = ops.bmm_nt(a, b_, 0.5, d, 2.0)
    want = 0.5 * a.float() @ b_.float().transpose(1, 2) + 2.0 * d.float()
    torch.cuda.synchronize()
    _status_ok()
    _close(out, want, 0.15, 2e-2)
    # transpose-free modes and their gradients
    kn = torch.randn(6, 256, 192, device=DEV, dtype=torch.bfloat16, requires_grad=True)      # [B, K, N]
    ar = a.detach().clone().requires_grad_(True)
    c1 = ops.bmm(ar, kn, 1)
    ar32, kn32 = ar.detach().float().requires_grad_(True), kn.detach().float().requires_grad_(True)
    c1r = ar32 @ kn32
    _close(c1, c1r, 0.3, 2e-2, "nn")
    gc = torch.randn_like(c1)
    g1, g2 = torch.autograd.grad(c1, [ar, kn], gc)
    g1r, g2r = torch.autograd.grad(c1r, [ar32, kn32], gc.float())
    _close(g1, g1r, 0.4, 3e-2, "nn dA")
    _close(g2, g2r, 0.4, 3e-2, "nn dB")
    km = torch.randn(6, 256, 128, device=DEV, dtype=torch.bfloat16)                           # [B, K, M]
    c2 = ops.bmm(km, kn.detach(), 2)
    _close(c2, km.float().transpose(1, 2) @ kn.detach().float(), 0.3, 2e-2, "tn")
    torch.cuda.synchronize()
    _status_ok()
    for shape in ((5, 384, 128), (3, 128, 384)):
        gg = torch.randn(*shape, device=DEV)
        xx = ops.newton_schulz(gg)
        xr_ = ref.newton_schulz(gg.cpu(), compute_dtype=torch.float32)
        _close(xx.cpu(), xr_, 6e-2, 6e-2, f"ns {shape}")
    g = torch.randn(5, 384, 128, device=DEV)
    x = ops.newton_schulz(g)
    xr = ref.newton_schulz(g.cpu(), compute_dtype=torch.float32)
    _close(x.cpu(), xr, 6e-2, 6e-2)
    s = torch.linalg.svdvals(x.float())
    assert s.max() < 1.3 and s.min() > 0.5


def test_adamw_flat_matches_torch():
    ext = _ext()
    torch.manual_seed(9)
    n = 8 * 1000
    p = torch.randn(n, device=DEV)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    plow = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    one = torch.ones(1, device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV)
        ref_p.grad = g.clone()
        opt.step()
        ext.adamw_flat(p, g.bfloat16().float(), m, v, plow, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, one, one, 1.0, n)
    _close(p, ref_p.detach(), 2e-3, 2e-3)
    _close(plow, p, 1e-2, 1e-2)
    # apply == 0 leaves everything untouched
    before = p.clone()
    ext.adamw_flat(p, torch.randn(n, device=DEV), m, v, plow, 1e-2, 0.9, 0.95, 1e-8, 0.1, 5, one, one * 0, 1.0, n)
    _close(p, before, 0, 0)
    out = torch.zeros(1, device=DEV)
    gg = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    ext.sumsq_accum(gg, 0.5, out)
    _close(out[0], (gg.float() * 0.5).pow(2).sum(), 1e-1, 1e-3)


@pytest.mark.parametrize("v", [1000, 12000, 32000, 50264, 33001])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy_in_place_kernel(v, dtype):
    """softmax(logits) - onehot in place and the summed loss, for row lengths that take the register-resident
    kernel (2, 4 or 8 vectors per thread) and the streaming kernel (rows too long or not a multiple of 8)."""
    ext = _ext()
    torch.manual_seed(12)
    t = 37
    logits = (torch.randn(t, v, device=DEV) * 3).to(dtype)
    labels = torch.randint(0, v, (t,), device=DEV)
    labels[5] = -100
    labels[6] = v - 1
    want = torch.softmax(logits.float(), -1)
    keep = labels != -100
    want[keep, labels[keep]] -= 1
    want[~keep] = 0
    want_loss = F.cross_entropy(logits.float(), labels, ignore_index=-100, reduction="sum")
    loss = torch.zeros(1, device=DEV)
    work = logits.clone()
    ext.ce_fwd_bwd_(work, labels, loss, -100)
    _close(work, want, 4e-3 if dtype == torch.bfloat16 else 1e-6, 1e-2 if dtype == torch.bfloat16 else 1e-4, "grad")
    _close(loss[0], want_loss, 1e-2, 1e-4, "loss")


def test_linear_cross_entropy():
    _ext()
    torch.manual_seed(10)
    t, d, v = 1000, 128, 32000
    h = (torch.randn(t, d, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(v, d, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    labels = torch.randint(0, v, (t,), device=DEV)
    labels[::7] = -100
    loss = ops.linear_cross_entropy(h, w, labels, chunk=256)
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lossr = F.cross_entropy(hr @ wr.t(), labels, ignore_index=-100)
    _close(loss, lossr, 2e-2, 1e-2)
    loss.backward()
    lossr.backward()
    _close(h.grad, hr.grad, 1e-4, 5e-2)
    _close(w.grad, wr.grad, 1e-4, 5e-2)


@pytest.mark.parametrize("hd,lq,lk,window,causal", [(64, 256, 256, 128, True), (96, 384, 700, 200, True),
                                                     (128, 128, 128, None, True), (96, 2048, 4095, 2048, True),
                                                     (64, 1024, 1024, None, False)])
def test_swa_attention_forward_backward(hd, lq, lk, window, causal):
    _ext()
    torch.manual_seed(11)
    b, h = 2, 3
    q = torch.randn(b, lq, h, hd, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, lk, h, hd, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, lk, h, hd, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = ops.swa_attention(q, k, v, window, causal=causal)
    torch.cuda.synchronize()
    _status_ok()
    qr, kr, vr = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    orf = ref.swa_attention(qr, kr, vr, window, causal=causal)
    _close(o, orf, 2e-2, 2e-2, "out")
    g = torch.randn_like(o)
    gq, gk, gv = torch.autograd.grad(o, [q, k, v], g)
    gqr, gkr, gvr = torch.autograd.grad(orf, [qr, kr, vr], g.float())
    _close(gq, gqr, 5e-2, 5e-2, "dq")
    _close(gk, gkr, 5e-2, 5e-2, "dk")
    _close(gv, gvr, 5e-2, 5e-2, "dv")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_patch_decode_matches_reference(dtype):
    _ext()
    torch.manual_seed(23)
    b, v, h, w, p = 2, 3, 32, 48, 8
    t = (h // p) * (w // p)
    y = torch.randn(b, v * t, p * p * 3, device=DEV).to(dtype).requires_grad_(True)
    target = torch.rand(b, v, 3, h, w, device=DEV)
    r, sse = ops.patch_decode(y, target, v, h, w, p)
    yr = y.detach().float().requires_grad_(True)
    rr = torch.sigmoid(yr).view(b, v, h // p, w // p, p, p, 3).permute(0, 1, 6, 2, 4, 3, 5).reshape(b, v, 3, h, w)
    sser = ((rr - target) ** 2).sum(dim=(2, 3, 4))
    _close(r, rr, 1e-5, 1e-5, "rendering")
    _close(sse, sser, 1e-2, 1e-4, "sse")
    gr = torch.randn_like(r)
    gs = torch.randn_like(sse)
    (g,) = torch.autograd.grad([r, sse], y, [gr, gs])
    (gref,) = torch.autograd.grad([rr, sser], yr, [gr, gs])
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(g, gref, tol, tol, "dy")


def test_fanout_and_stacked_linear_accumulate_gradients_in_the_gemm():
    _ext()
    torch.manual_seed(24)
    x = torch.randn(4, 64, 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    flat = (torch.randn(3 * 256 * 128, device=DEV) * 0.05).bfloat16()
    gflat = torch.zeros_like(flat)
    ws = []
    for i in range(3):                                   # three neighbours in one flat buffer, like the trainer's
        w = flat[i * 256 * 128:(i + 1) * 256 * 128].view(256, 128).requires_grad_(True)
        w.grad = gflat[i * 256 * 128:(i + 1) * 256 * 128].view(256, 128)
        w.grad.fill_(0.5)
        ws.append(w)
    ops.set_fused_weight_grad(True)
    try:
        a, b = ops.fanout_linear(x, ws[:2])
        c = ops.stacked_linear(x, ws[1], ws[2])
        ga, gb, gc = torch.randn_like(a), torch.randn_like(b), torch.randn_like(c)
        (a * ga).sum().add((b * gb).sum()).add((c * gc).sum()).backward()
    finally:
        ops.set_fused_weight_grad(False)
    xr = x.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    ar, br = xr @ wr[0].t(), xr @ wr[1].t()
    cr = xr @ torch.cat([wr[1], wr[2]]).t()
    _close(a, ar, 3e-2, 3e-2, "a")
    _close(c, cr, 3e-2, 3e-2, "c")
    (ar * ga.float()).sum().add((br * gb.float()).sum()).add((cr * gc.float()).sum()).backward()
    _close(x.grad, xr.grad, 0.15, 3e-2, "dx")
    for i in range(3):
        _close(ws[i].grad, 0.5 + wr[i].grad, 0.6, 3e-2, f"dw{i}")        # added onto the existing 0.5
    assert gflat.view(3, 256, 128)[0].data_ptr() == ws[0].grad.data_ptr()  # still the flat buffer's view


def test_grad_sink_matches_autograd_accumulation():
    _ext()
    torch.manual_seed(25)
    plan = _plan(seed=3)
    g, k, n = plan.num_groups, 128, 256
    real = torch.zeros(plan.rows_padded, 1, device=DEV)
    real[plan.dest.reshape(-1)] = 1
    xs = [(torch.randn(plan.rows_padded, k, device=DEV) * real).bfloat16() for _ in range(3)]
    cs = [(torch.randn(plan.rows_padded, n, device=DEV) * real).bfloat16() for _ in range(3)]

    def run(use_sink):
        w = (torch.randn(g, n, k, device=DEV, generator=torch.Generator(DEV).manual_seed(1)) / 11).bfloat16()
        w.requires_grad_(True)
        ws = ops.grad_sink(w * 1.0) if use_sink else w * 1.0     # a non-leaf, like a chunk's state
        total = 0
        for x, c in zip(xs, cs):
            total = total + (ops.gg_nt(x, ws, plan).float() * c.float()).sum()
        # one consumer that knows nothing about sinks contributes through autograd as usual
        total = total + (ws.float() ** 2).sum() * 0.01
        total.backward()
        return w.grad.float()

    a, b = run(False), run(True)
    # autograd sums the three bf16 contributions in bf16, the sink in fp32: equal up to bf16 rounding of sums ~10
    _close(b, a, 1.0, 3e-2, "sink")
    assert not fn._GRAD_SINKS


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_frobenius_normalize_forward_backward(dtype):
    ext = _ext()
    torch.manual_seed(26)
    g = (torch.randn(5, 384, 128, device=DEV) * 3).to(dtype).requires_grad_(True)
    x = fn._FrobNormalize.apply(g, 1e-7)
    gr = g.detach().float().requires_grad_(True)
    xr = gr / (gr.norm(dim=(1, 2), keepdim=True) + 1e-7)
    _close(x, xr, 1e-3, 1e-2, "x")
    c = torch.randn_like(xr).bfloat16()
    (d,) = torch.autograd.grad(x, g, c)
    (dr,) = torch.autograd.grad(xr, gr, c.float())
    _close(d, dr, 2e-3 if dtype == torch.float32 else 2e-2, 2e-2, "dg")


def test_activation_offload_round_trip():
    _ext()
    from uttt_b200.utils.activation_offload import offload_activations
    torch.manual_seed(27)
    lin = torch.nn.Linear(256, 256).to(DEV)
    x = torch.randn(512, 256, device=DEV, requires_grad=True)
    ref_out = (lin(x).relu() ** 2).sum()
    (gref,) = torch.autograd.grad(ref_out, x)
    with offload_activations(min_bytes=1024) as off:
        out = (lin(x).relu() ** 2).sum()
    (g,) = torch.autograd.grad(out, x)
    assert off.tensors_offloaded > 0 and off.bytes_offloaded >= 512 * 256 * 4
    _close(g, gref, 0, 0, "grad through offloaded activations")


def test_plucker_embed():
    _ext()
    from uttt_b200.nvs.data import SyntheticScenes
    batch = {k: v.to(DEV) for k, v in next(SyntheticScenes(2, 3, 64, pin=False)).items()}
    tgt = torch.tensor([False, True, False], device=DEV)
    got = ops.plucker_embed(batch["image"], batch["fxfycxcy"], batch["c2w"], tgt, 8)
    want = ref.plucker_embed(batch["image"], batch["fxfycxcy"], batch["c2w"], tgt, 8)
    _close(got, want, 1e-5, 1e-5)


def test_tiny_lm_gpu_matches_cpu():
    """Whole-model check: bf16 kernels on the GPU against the fp32 CPU path, same weights."""
    _ext()
    from uttt_b200.config import named_config
    from uttt_b200.models import build_model
    torch.manual_seed(0)
    cfg = named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                       memory_num_active_experts=2, chunk_size=128, window_size=128, memory_lb_loss_alpha=0.0)
    model = build_model(cfg)
    ids = torch.randint(0, 1024, (2, 512))
    out_cpu = model(input_ids=ids, labels=ids)
    out_cpu.loss.backward()
    gcpu = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    gm = build_model(cfg)
    gm.load_state_dict(model.state_dict())
    gm = gm.to(DEV).to(torch.bfloat16)
    out_gpu = gm(input_ids=ids.to(DEV), labels=ids.to(DEV))
    out_gpu.loss.backward()
    torch.cuda.synchronize()
    _status_ok()
    assert abs(out_gpu.loss.item() - out_cpu.loss.item()) < 0.05
    cosines = {}
    for n, p in gm.named_parameters():
        a, b_ = p.grad.float().cpu(), gcpu[n]
        if b_.abs().max() < 1e-6 or b_.numel() < 8:   # a scalar's cosine is only its sign
            continue
        cosines[n] = float(F.cosine_similarity(a.flatten(), b_.flatten(), dim=0))
    # bf16 end to end: nearly all gradients line up tightly; the tiny second-order ones (learning-rate and
    # momentum heads) are noisier but must still point the same way
    good = sum(c > 0.9 for c in cosines.values())
    assert good >= 0.85 * len(cosines), sorted(cosines.items(), key=lambda kv: kv[1])[:8]
    assert min(cosines.values()) > 0.5, sorted(cosines.items(), key=lambda kv: kv[1])[:8]


def _gpu_vs_cpu_lm(cfg, seq=256, loss_tol=0.06, frac=0.8):
    from uttt_b200.models import build_model
    torch.manual_seed(0)
    model = build_model(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, seq))
    out_cpu = model(input_ids=ids, labels=ids)
    out_cpu.loss.backward()
    gcpu = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    gm = build_model(cfg)
    gm.load_state_dict(model.state_dict())
    gm = gm.to(DEV).to(torch.bfloat16)
    out_gpu = gm(input_ids=ids.to(DEV), labels=ids.to(DEV))
    out_gpu.loss.backward()
    torch.cuda.synchronize()
    _status_ok()
    assert abs(out_gpu.loss.item() - out_cpu.loss.item()) < loss_tol, (out_gpu.loss.item(), out_cpu.loss.item())
    cos = {}
    for n, p in gm.named_parameters():
        if n not in gcpu or p.grad is None or gcpu[n].numel() < 8 or gcpu[n].abs().max() < 1e-6:
            continue
        cos[n] = float(F.cosine_similarity(p.grad.float().cpu().flatten(), gcpu[n].flatten(), dim=0))
    good = sum(c > 0.9 for c in cos.values())
    assert good >= frac * len(cos), sorted(cos.items(), key=lambda kv: kv[1])[:8]


@pytest.mark.parametrize("family", ["uttt_dense", "ttt_moe_lb", "ttt_dense"])
def test_other_families_gpu_match_cpu(family):
    """The dense and layer-local families run through the same kernels: GPU bf16 against the fp32 CPU path."""
    _ext()
    from uttt_b200.config import config_from_dict
    base = dict(model_type=family, hidden_size=256, num_hidden_layers=2, num_heads=4, fw_num_heads=2, vocab_size=1024,
                chunk_size=128, window_size=128, memory_kv_mode="reuse_kv", use_momentum=True, use_moun=True,
                w0_w2_low_rank=0)
    if family == "ttt_moe_lb":
        base.update(memory_num_experts=4, memory_num_active_experts=2)
    _gpu_vs_cpu_lm(config_from_dict(base))


def test_lvsm_gpu_matches_cpu():
    """View-synthesis model end to end on the GPU (Plucker embed, memory blocks, fused decoder tail) against CPU."""
    _ext()
    from uttt_b200.nvs.data import SyntheticScenes
    from uttt_b200.nvs.model import LVSMModel
    p = dict(attn_head_dim=32, fw_head_dim=64, inter_multi=2, fw_inter_multi=2, use_muon=True, num_experts=4,
             num_active_experts=2, l2_norm=True, pool_mode="shared", router_share_mode="share_all", aggregate_write=True,
             load_balancing_loss_alpha=1e-5)
    cfg = {"exp_name": "t", "model": {"image_size": 64, "patch_size": 8, "dim": 128, "layers": 2,
                                      "block_config": {"type": "uttt_nvs.models.uttt_moe_block.MemoryModel",
                                                       "params": p}},
           "training": {"num_views": 4}}
    torch.manual_seed(0)
    m = LVSMModel(cfg)
    batch = next(SyntheticScenes(2, 4, 64, pin=False))
    out = m(batch)
    out["loss_metrics"]["loss"].backward()
    g = LVSMModel(cfg)
    g.load_state_dict(m.state_dict())
    g = g.to(DEV).to(torch.bfloat16)
    outg = g({k: v.to(DEV) for k, v in batch.items()})
    outg["loss_metrics"]["loss"].backward()
    torch.cuda.synchronize()
    _status_ok()
    assert abs(float(outg["loss_metrics"]["loss"]) - float(out["loss_metrics"]["loss"])) < 0.02
    _close(outg["rendering"].cpu(), out["rendering"], 0.06, 0.0, "rendering")
    cos = []
    for (n, a), (_, b_) in zip(g.named_parameters(), m.named_parameters()):
        if a.grad is None or b_.grad is None or b_.grad.numel() < 8 or b_.grad.abs().max() < 1e-7:
            continue
        cos.append(float(F.cosine_similarity(a.grad.float().cpu().flatten(), b_.grad.flatten(), dim=0)))
    assert sum(c > 0.9 for c in cos) >= 0.75 * len(cos), sorted(cos)[:8]


def test_cached_generation_on_gpu_matches_one_shot_forward():
    """Incremental decoding through the kernels (single-token attention calls, routing of one row per head)."""
    _ext()
    from uttt_b200.config import named_config
    from uttt_b200.models import build_model
    from uttt_b200.models.generation import generate
    torch.manual_seed(0)
    cfg = named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                       memory_num_active_experts=2, chunk_size=64, window_size=64)
    model = build_model(cfg).to(DEV).to(torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (1, 160), device=DEV)
    with torch.no_grad():
        full = model(input_ids=ids).logits.float()
        out = model(input_ids=ids[:, :100], use_cache=True)
        parts = [out.logits.float()]
        cache = out.past_key_values
        for t in range(100, 160):
            out = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            cache = out.past_key_values
            parts.append(out.logits.float())
    got = torch.cat(parts, dim=1)
    torch.cuda.synchronize()
    _status_ok()
    assert torch.isfinite(got).all()
    # bf16 end to end: compare the distributions, not the raw logits
    agree = (got.argmax(-1) == full.argmax(-1)).float().mean().item()
    assert agree > 0.9, agree
    diff = (torch.log_softmax(got, -1) - torch.log_softmax(full, -1)).abs()
    # a near-tied router logit may pick another expert for a token in one of the two passes: a handful of entries
    assert float((diff > 0.25).float().mean()) < 1e-4 and float(diff.max()) < 0.75, (float(diff.max()),)
    toks = generate(model, ids[:, :10], max_new_tokens=5)
    assert toks.shape == (1, 15)


@pytest.mark.parametrize("mode", ["cross_layer_cut", "first_order_state", "stop_state"])
def test_backward_modes_gpu_match_cpu(mode):
    _ext()
    from uttt_b200.config import named_config
    cfg = named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                       memory_num_active_experts=2, chunk_size=128, window_size=128, memory_lb_loss_alpha=0.0,
                       memory_update_backward_mode=mode)
    _gpu_vs_cpu_lm(cfg, seq=384, frac=0.75)


def test_bounded_wait_gives_up_records_status_and_next_launch_is_healthy():
    """A consumer that waits for a block nobody announces must give up after its limit, record status 51, return with
    its tensor memory freed, and leave the device usable: the next launch (status word cleared) is correct.
    One GPU plays both ranks of the gather-fused GEMM: the 'peer' shard is a second buffer on the same device, and
    the gather CTAs of the SAME launch copy it but withhold the announcement (nothing faults, traps or hangs)."""
    import time
    ext = _ext()
    torch.manual_seed(31)
    m, k, n = 256, 128, 1024
    x = torch.randn(m, k, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) / math.sqrt(k)).bfloat16()
    want = x.float() @ w.float().t()
    peer = w[n // 2:].clone()                                 # the other rank's rows
    w_full = torch.zeros_like(w)
    w_full[:n // 2] = w[:n // 2]                              # this rank's rows are in place
    ptrs = [w_full.data_ptr(), peer.data_ptr()]
    ready = torch.zeros(n // 256, dtype=torch.int32, device=DEV)
    status = ext.gemm_status(x)
    status.zero_()
    out = ext.ag_linear(x, ptrs, 0, w_full, ready, 8)
    torch.cuda.synchronize()
    _status_ok()
    _close(out, want, 3e-2, 3e-2, "healthy launch")
    # the peer's blocks are never announced: the wait runs out after 5 ms
    w_full[n // 2:] = 0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ext.ag_linear(x, ptrs, 0, w_full, ready, 8, wait_limit_ms=5.0, withhold_from_block=(n // 256) // 2)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert int(status[0].item()) == 51, int(status[0].item())
    assert elapsed < 1.0, f"the kernel took {elapsed:.3f} s to give up on a 5 ms limit"
    # while the word is set, tensor-core kernels return at once; after clearing it everything works again
    status.zero_()
    w_full[n // 2:] = 0
    out = ext.ag_linear(x, ptrs, 0, w_full, ready, 8)
    torch.cuda.synchronize()
    _status_ok()
    _close(out, want, 3e-2, 3e-2, "launch after the failed wait")
    a = torch.randn(256, 128, device=DEV, dtype=torch.bfloat16)
    _close(ops.bmm_nt(a[None], a[None]), (a.float() @ a.float().t())[None], 0.2, 3e-2, "tcgen05 GEMM after it")
    _status_ok()


def test_training_step_is_reproducible_run_to_run():
    """Same seed, same data, twice.  A race between kernels (a consumer that starts before its producer's data is
    complete, a staging slab reused too early) shows up as gross differences.  What is legitimately unordered is a
    handful of fp32 atomic sums (loss, gradient norm, router probability sums, the q/k scale gradients, the Frobenius
    norms, the embedding-gradient scatter): they move results by fp32 rounding, which can flip the bf16 rounding of
    a few parameter elements by one unit in the last place."""
    _ext()
    from uttt_b200.config import named_config
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    cfg = named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                       memory_num_active_experts=2, chunk_size=128, window_size=128)
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(5))
    runs = []
    for _ in range(2):
        eng = TrainEngine(cfg, EngineConfig(micro_batch_size=2, warmup_steps=0, total_steps=4, seed=3),
                          torch.device(DEV, 0))
        losses = [float(eng.train_step({"input_ids": ids, "labels": ids})) for _ in range(2)]
        torch.cuda.synchronize()
        masters = eng.trainer.optimizer_state_dict()["state"]
        runs.append((losses, {k: v["master"].float() for k, v in masters.items()}))
    _status_ok()
    # a flipped bf16 rounding of the Newton-Schulz input (its Frobenius norm is an atomic fp32 sum) changes a few
    # fast-weight entries by 2^-8 relative; on the loss that is ~1e-5 relative.  A race would be orders above it.
    # (the second step starts from weights that already differ in their last bits, and near-tied router logits
    # then pick other experts for a few tokens: a few 1e-4 relative on its loss)
    for a, b_, tol in zip(runs[0][0], runs[1][0], (2e-4, 1e-3)):
        assert abs(a - b_) <= tol * abs(a), (runs[0][0], runs[1][0])
    for k, v in runs[0][1].items():
        w = runs[1][1][k]
        # fp32 masters after two AdamW steps: update size lr = 1e-3 per step; a differing sign of a near-zero
        # gradient moves an element by at most 2 lr per step
        # Gradients that are sums over all tokens with heavy cancellation (norm weights, biases) move by a few
        # percent from those flips; with lr = 1e-3 that is ~1e-5 on a master, against ~1e-3 if a kernel had read
        # data that was not there yet.
        diff = (v - w).abs()
        assert float(diff.max()) <= 4.5e-3, (k, float(diff.max()))
        assert float(diff.mean()) <= 1.5e-4, (k, float(diff.mean()))


def test_dense_projections_on_the_own_kernel_match_fp32():
    """``set_dense_gemm(True)``: fan-out and stacked linears run forward, input gradient and weight gradient on the
    batched tcgen05 kernel; compared with fp32 PyTorch and with the library route."""
    from uttt_b200 import ops
    torch.manual_seed(0)
    dev = torch.device("cuda", 0)
    x = (torch.randn(4, 256, 384, device=dev) * 0.5).bfloat16().requires_grad_(True)
    ws = [(torch.randn(n, 384, device=dev) * 0.05).bfloat16().requires_grad_(True) for n in (384, 128, 64)]
    bias = (torch.randn(64, device=dev) * 0.1).bfloat16().requires_grad_(True)
    wa, wb = [(torch.randn(512, 384, device=dev) * 0.05).bfloat16().requires_grad_(True) for _ in range(2)]

    def run():
        ys = ops.fanout_linear(x, ws, [None, None, bias])
        z = ops.stacked_linear(x, wa, wb)
        loss = sum((y.float() ** 2).sum() for y in ys) + (z.float() * 0.5).sum()
        grads = torch.autograd.grad(loss, [x, *ws, bias, wa, wb])
        return [y.detach() for y in ys] + [z.detach()], grads

    xf = x.detach().float().requires_grad_(True)
    wsf = [w.detach().float().requires_grad_(True) for w in ws]
    bf_, waf, wbf = (t.detach().float().requires_grad_(True) for t in (bias, wa, wb))
    ysf = [torch.nn.functional.linear(xf, w, b) for w, b in zip(wsf, [None, None, bf_])]
    zf = torch.nn.functional.linear(xf, torch.cat([waf, wbf], 0))
    lossf = sum((y ** 2).sum() for y in ysf) + (zf * 0.5).sum()
    gradsf = torch.autograd.grad(lossf, [xf, *wsf, bf_, waf, wbf])
    try:
        ops.set_dense_gemm(True)
        before = ops.launch_count()
        outs, grads = run()
        # 4 forward, 4 input-gradient and 3 weight-gradient products (the 64-row weight gradient is below the
        # kernel's 128-row tile and stays on the library)
        assert ops.launch_count() - before >= 11
    finally:
        ops.set_dense_gemm(False)
    outs_lib, grads_lib = run()

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))
    for got, lib, want in zip(outs, outs_lib, ysf + [zf]):
        assert rel(got, want) < 6e-3 and rel(got, lib) < 6e-3
    for got, lib, want in zip(grads, grads_lib, gradsf):
        assert rel(got, want) < 1.2e-2 and rel(got, lib) < 1.2e-2, (rel(got, want), rel(got, lib))


def _one_rank_ep_plan(idx, experts):
    """The expert-parallel layout of a group of one rank (owner = sender), from the same kernels a real group uses."""
    from uttt_b200 import ops
    ext = _ext()
    bsz, n, k = idx.shape
    local = ops.build_group_plan(idx, experts)
    sizes32 = local.sizes.to(torch.int32).contiguous()
    want = 2 * bsz * n * k
    cap_rows = ((want + 127) // 128 + bsz * experts) * 128
    remote_start, tile_group, offsets, sizes = ext.ep_plan(sizes32.view(1, -1), 0, bsz, experts, cap_rows // 128)
    return local, sizes32, remote_start, tile_group, offsets, cap_rows


def test_tile_driven_expert_parallel_read_on_one_rank():
    """push (with per-tile row counters) -> gate|up GEMM that waits for complete tiles -> down GEMM that reports
    finished tiles -> pull that waits for them: the whole chain on a group of one rank, against the plain kernels
    and fp32."""
    from uttt_b200 import ops
    ext = _ext()
    torch.manual_seed(0)
    bsz, n, k, experts, d, inter = 2, 1024, 2, 4, 128, 256
    idx = torch.randint(0, experts, (bsz, n, k), device=DEV)
    idx[..., 1] = (idx[..., 0] + 1 + torch.randint(0, experts - 1, (bsz, n), device=DEV)) % experts
    local, sizes32, remote_start, tile_group, offsets, cap_rows = _one_rank_ep_plan(idx, experts)
    rows = (torch.randn(bsz * n, d, device=DEV) * 0.5).bfloat16()
    wts = torch.rand(bsz * n, k, device=DEV)
    w02 = (torch.randn(bsz * experts, 2 * inter, d, device=DEV) * 0.1).bfloat16()
    w1 = (torch.randn(bsz * experts, d, inter, device=DEV) * 0.1).bfloat16()
    tiles = cap_rows // 128
    recv = torch.full((cap_rows, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    send = torch.full((cap_rows, d), float("nan"), device=DEV, dtype=torch.bfloat16)
    ready = torch.zeros(tiles, device=DEV, dtype=torch.int32)
    done = torch.zeros(tiles, device=DEV, dtype=torch.int32)
    idx32 = idx.reshape(bsz * n, k).to(torch.int32).contiguous()
    maps = (idx32, local.dest.contiguous(), local.offsets)
    per_tile = int(ext.gg_nt_done_per_tile(d))
    for use in (1, 2):                                     # the send counters only grow: second use, second target
        ext.ep_push(rows, None, *maps, sizes32, remote_start, [recv.data_ptr()], experts, n, cap_rows,
                    [ready.data_ptr()])
        used = tile_group >= 0
        assert bool((ready[used] == 128).all()) and bool((ready[~used] == 0).all())
        hid = ext.gg_nt_swiglu(recv, w02, tile_group, ready, 128, 50.0)
        ready.zero_()
        ext.gg_nt(hid, w1, tile_group, send, None, 0, done, 50.0)
        assert bool((done == use * per_tile).all())        # every tile reports, used or not
        y = ext.ep_pull([send.data_ptr()], wts, *maps, remote_start, experts, n, d, torch.bfloat16, cap_rows,
                        [done.data_ptr()], use * per_tile, 50.0)
        _status_ok()
        # oracle: per routed copy in fp32
        g = (torch.arange(bsz, device=DEV).repeat_interleave(n)[:, None] * experts + idx.reshape(-1, k))
        xf = rows.float()
        want = torch.zeros(bsz * n, d, device=DEV)
        for j in range(k):
            w02j, w1j = w02[g[:, j]].float(), w1[g[:, j]].float()
            y02 = torch.einsum("rnd,rd->rn", w02j, xf)
            h = (torch.nn.functional.silu(y02[:, :inter]) * y02[:, inter:]).bfloat16().float()
            want += wts[:, j:j + 1] * torch.einsum("rdi,ri->rd", w1j, h).bfloat16().float()
        rel = float((y.float() - want).norm() / want.norm())
        assert rel < 1e-2, rel


def test_tile_driven_read_waits_run_out_with_a_status():
    """Counters that nothing completes: the producer of the gate|up GEMM and the pulling warps give up after a few
    milliseconds, report 62 / 63 in the status word and return; the kernels work again once the word is cleared."""
    ext = _ext()
    torch.manual_seed(0)
    bsz, n, k, experts, d, inter = 1, 512, 2, 2, 128, 256
    idx = torch.stack([torch.zeros(bsz, n, dtype=torch.long), torch.ones(bsz, n, dtype=torch.long)], -1).to(DEV)
    local, sizes32, remote_start, tile_group, offsets, cap_rows = _one_rank_ep_plan(idx, experts)
    tiles = cap_rows // 128
    x = torch.randn(cap_rows, d, device=DEV).bfloat16()
    w02 = (torch.randn(bsz * experts, 2 * inter, d, device=DEV) * 0.1).bfloat16()
    never = torch.zeros(tiles, device=DEV, dtype=torch.int32)
    st = ext.gemm_status(torch.zeros(1, device=DEV))
    st.zero_()
    ext.gg_nt_swiglu(x, w02, tile_group, never, 128, 5.0)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 62
    st.zero_()
    idx32 = idx.reshape(bsz * n, k).to(torch.int32).contiguous()
    ext.ep_pull([x.data_ptr()], None, idx32, local.dest.contiguous(), local.offsets, remote_start, experts, n, d,
                torch.bfloat16, cap_rows, [never.data_ptr()], 8, 5.0)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 63
    st.zero_()
    full = torch.full((tiles,), 128, device=DEV, dtype=torch.int32)
    got = ext.gg_nt_swiglu(x, w02, tile_group, full, 128, 5.0)
    want = ext.gg_nt_swiglu(x, w02, tile_group)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    _status_ok()


def _checked_build() -> bool:
    import uttt_b200.ops as ops_pkg
    marker = os.path.join(os.path.dirname(ops_pkg.__file__), "_C.so.flavour")
    try:
        with open(marker) as fh:
            return fh.read().strip() == "checked"
    except OSError:
        return False


def test_checked_build_reports_bad_indices_instead_of_following_them():
    """Only in the checked build (``UTTT_B200_BOUNDS_CHECK=1 python -m uttt_b200.ops.build``): an index table that points
    outside its buffer is reported through the status word and the access is skipped.  The regular build does not
    carry the checks, so this test does not run there."""
    if not _checked_build():
        pytest.skip("the loaded extension is the regular build")
    from uttt_b200 import ops
    ext = _ext()
    st = ext.gemm_status(torch.zeros(1, device=DEV))
    st.zero_()
    idx = torch.randint(0, 4, (1, 256, 2), device=DEV)
    plan = ops.build_group_plan(idx, 4)
    x = torch.randn(256, 128, device=DEV, dtype=torch.bfloat16)
    good = ops.permute_rows(x, plan)
    bad_dest = plan.dest.clone()
    bad_dest[3, 1] = plan.rows_padded + 5                      # past the end of the permuted buffer
    bad = ops.GroupPlan(bad_dest, plan.offsets, plan.sizes, plan.tile_group, plan.rows_padded, plan.num_groups, 2)
    ops.permute_rows(x, bad)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 71
    st.zero_()
    ops.unpermute_rows(good, bad, torch.ones(256, 2, device=DEV))
    torch.cuda.synchronize()
    assert int(st[0].item()) == 72
    st.zero_()
    w = torch.randn(4, 256, 128, device=DEV, dtype=torch.bfloat16)
    tiles = plan.tile_group.clone()
    tiles[0] = 9                                               # a group the weights do not have
    out = ext.gg_nt(good, w, tiles)
    torch.cuda.synchronize()
    assert int(st[0].item()) == 74
    assert float(out[:128].abs().max()) == 0.0                 # the tile was treated as unused (zero filled)
    st.zero_()
    want = ext.gg_nt(good, w, plan.tile_group)
    torch.cuda.synchronize()
    assert torch.equal(out[128:], want[128:])
    _status_ok()


def test_split_linear_matches_fp32():
    """One q|k|v weight, three contiguous outputs; input gradient accumulated in the GEMMs, weight gradient written
    block by block."""
    from uttt_b200 import ops
    torch.manual_seed(0)
    x = (torch.randn(2, 256, 192, device=DEV) * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(3 * 192, 192, device=DEV) * 0.05).bfloat16().requires_grad_(True)
    q, k, v = ops.split_linear(x, w, 3)
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and q.shape == (2, 256, 192)
    loss = (q.float() * 1.0).pow(2).sum() + (k.float() * 2.0).sum() + (v.float().pow(3)).sum()
    dx, dw = torch.autograd.grad(loss, [x, w])
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    qf, kf, vf = torch.nn.functional.linear(xf, wf).chunk(3, dim=-1)
    lossf = qf.pow(2).sum() + (kf * 2.0).sum() + vf.pow(3).sum()
    dxf, dwf = torch.autograd.grad(lossf, [xf, wf])

    def rel(a, b):
        return float((a.float() - b).norm() / b.norm())
    assert rel(q, qf) < 6e-3 and rel(k, kf) < 6e-3 and rel(v, vf) < 6e-3
    assert rel(dx, dxf) < 1.2e-2 and rel(dw, dwf) < 1.2e-2, (rel(dx, dxf), rel(dw, dwf))
    # only one of the three outputs used: the other blocks of the weight gradient are zero
    q2, _, _ = ops.split_linear(x, w, 3)
    (dw2,) = torch.autograd.grad(q2.float().sum(), [w])
    assert float(dw2[192:].abs().max()) == 0.0 and float(dw2[:192].abs().max()) > 0.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rms_norm_gated_matches_fp32(dtype):
    """Per-head norm of the memory read with its gate in the same kernel; gate gradient from the norm's backward."""
    from uttt_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(3, 70, 4, 384, device=DEV, dtype=dtype, requires_grad=True)
    w = (torch.randn(384, device=DEV) * 0.1 + 1).to(dtype).requires_grad_(True)
    gate = torch.randn(3, 70, 4, device=DEV, dtype=dtype, requires_grad=True)
    y = ops.rms_norm_gated(x, w, gate, 1e-5)
    dy = torch.randn_like(y)
    gx, gw, gg = torch.autograd.grad(y, [x, w, gate], dy)
    xf, wf, gf = (t.detach().float().requires_grad_(True) for t in (x, w, gate))
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf * gf.unsqueeze(-1)
    fx, fw_, fg = torch.autograd.grad(yf, [xf, wf, gf], dy.float())

    def rel(a, b):
        return float((a.float() - b).norm() / b.norm())
    tol = 6e-3 if dtype == torch.bfloat16 else 1e-5
    assert rel(y, yf) < tol and rel(gx, fx) < 2 * tol and rel(gw, fw_) < 2 * tol and rel(gg, fg) < 2 * tol, (
        rel(y, yf), rel(gx, fx), rel(gw, fw_), rel(gg, fg))


@pytest.mark.parametrize("shape", [(4, 384, 128), (4, 128, 384), (3, 256, 256)])
def test_newton_schulz_hand_written_backward(shape):
    """Gradient of the five Newton-Schulz iterations through the hand-written per-iteration backward (six batched GEMMs
    with accumulating epilogues), against fp32 autograd of the plain statement and against the autograd path through the
    individual batched GEMMs."""
    from uttt_b200.ops import functional as Fn
    torch.manual_seed(1)
    g = torch.randn(*shape, device=DEV, requires_grad=True)
    cot = torch.randn(*shape, device=DEV)

    def grad(fused):
        saved = Fn._NS_FUSED_BACKWARD
        Fn._NS_FUSED_BACKWARD = fused
        try:
            before = ops.launch_count()
            out = ops.newton_schulz(g)
            (dg,) = torch.autograd.grad(out, [g], cot.to(out.dtype))
            return out.detach().float(), dg.float(), ops.launch_count() - before
        finally:
            Fn._NS_FUSED_BACKWARD = saved

    out_f, dg_f, n_fused = grad(True)
    out_a, dg_a, n_auto = grad(False)
    gf = g.detach().float().requires_grad_(True)
    out_r = ref.newton_schulz(gf, compute_dtype=torch.float32)
    (dg_r,) = torch.autograd.grad(out_r, [gf], cot)
    torch.cuda.synchronize()
    _status_ok()

    def rel(a, b):
        return float((a - b).norm() / b.norm())
    # same forward kernels either way; the Frobenius norm is an atomic fp32 sum, so two runs differ in a few bf16 roundings
    assert rel(out_f, out_r) < 3e-2 and rel(out_f, out_a) < 1e-2
    # bf16 iterates: both kernel paths sit a few per cent from the fp32 gradient, and close to each other
    assert rel(dg_f, dg_r) < 6e-2 and rel(dg_a, dg_r) < 6e-2, (rel(dg_f, dg_r), rel(dg_a, dg_r))
    assert rel(dg_f, dg_a) < 4e-2, rel(dg_f, dg_a)
    assert n_fused <= n_auto                                               # never more launches of this extension
