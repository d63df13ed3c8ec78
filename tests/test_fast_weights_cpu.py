"""Grouped (tile-padded, expert-major) fast-weight path against a dense-mask einsum oracle.

The oracle restates the reference's per-(sequence, expert) loop semantics
(uttt_llm/flame/custom_models/uttt_moe/modeling_recurrent_lact.py:221-261, 389-451) with
masks instead of gathers; both are fp32 on CPU.
"""
import torch
import torch.nn.functional as F

from uttt_b200 import ops
from uttt_b200.config import named_config
from uttt_b200.models import fast_weights as fw
from uttt_b200.ops import reference as ref


def _setup(bsz=2, n=96, d=16, inter=24, e=4, k=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    rows = torch.randn(bsz, n, d, generator=g)
    w02 = torch.randn(bsz, e, 2 * inter, d, generator=g) / d ** 0.5
    w1 = torch.randn(bsz, e, d, inter, generator=g) / inter ** 0.5
    router = torch.randn(e, d, generator=g)
    cfg = named_config("tiny-uttt-moe", memory_num_experts=e, memory_num_active_experts=k)
    return rows, w02, w1, router, cfg


def _dense_read(rows, w02, w1, router, k):
    inter = w1.shape[-1]
    logits = rows @ router.t()
    probs = logits.softmax(-1)
    idx = logits.topk(k, -1).indices
    mask = torch.zeros_like(probs).scatter_(-1, idx, 1.0)
    w0, w2 = w02[:, :, :inter], w02[:, :, inter:]
    gate = torch.einsum("bnd,beid->beni", rows, w0)
    up = torch.einsum("bnd,beid->beni", rows, w2)
    out = torch.einsum("beni,bedi->bend", F.silu(gate) * up, w1)
    return (out * (probs * mask).permute(0, 2, 1).unsqueeze(-1)).sum(1)


def test_group_plan_layout():
    idx = torch.randint(0, 5, (3, 50, 2))
    plan = ops.build_group_plan(idx, 5)
    assert plan.rows_padded % ops.TILE_ROWS == 0
    assert int(plan.sizes.sum()) == idx.numel()
    offs = plan.offsets.tolist()
    assert all(o % ops.TILE_ROWS == 0 for o in offs)
    # every destination lies inside its group's real rows and destinations are unique
    gid = (idx + torch.arange(3)[:, None, None] * 5).reshape(-1)
    dest = plan.dest.reshape(-1)
    assert dest.unique().numel() == dest.numel()
    lo = plan.offsets[:-1].long()[gid]
    assert bool(((dest >= lo) & (dest < lo + plan.sizes.long()[gid])).all())
    # tile -> group table agrees with the offsets
    for t, g in enumerate(plan.tile_group.tolist()):
        start = t * ops.TILE_ROWS
        if g >= 0:
            assert offs[g] <= start < offs[g + 1]
        else:
            assert start >= offs[-1]


def test_pool_read_matches_dense_oracle():
    rows, w02, w1, router, cfg = _setup()
    rows.requires_grad_(True); w02.requires_grad_(True); w1.requires_grad_(True); router.requires_grad_(True)
    routing = fw.route_rows(rows, router, None, cfg)
    y = fw.pool_read(rows, w02, w1, routing)
    y_ref = _dense_read(rows, w02, w1, router, 2)
    torch.testing.assert_close(y, y_ref, atol=1e-4, rtol=1e-4)
    g = torch.randn_like(y)
    grads = torch.autograd.grad(y, [rows, w02, w1, router], g)
    grads_ref = torch.autograd.grad(y_ref, [rows, w02, w1, router], g)
    for a, b in zip(grads, grads_ref):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-3)


def _dense_raw_grad(k_rows, v_rows, lr_rows, w02, w1, router, k):
    inter = w1.shape[-1]
    logits = k_rows @ router.t()
    probs = logits.softmax(-1)
    idx = logits.topk(k, -1).indices
    mask = torch.zeros_like(probs).scatter_(-1, idx, 1.0)
    pw = (probs * mask).permute(0, 2, 1).unsqueeze(-1)              # [b,e,n,1]
    w0, w2 = w02[:, :, :inter], w02[:, :, inter:]
    gate = torch.einsum("bnd,beid->beni", k_rows, w0)
    up = torch.einsum("bnd,beid->beni", k_rows, w2)
    hidden = F.silu(gate) * up
    v = v_rows[:, None] * pw
    dhid = torch.einsum("bend,bedi->beni", v, w1)
    dup = dhid * F.silu(gate)
    dgate = ref.silu_backprop(dhid * up, gate)
    lr0, lr1, lr2 = [lr_rows[:, None, :, i:i + 1] for i in range(3)]
    g1 = torch.einsum("bend,beni->bedi", v, hidden * lr1)
    g0 = torch.einsum("beni,bend->beid", dgate, k_rows[:, None] * lr0 * (pw > 0))
    g2 = torch.einsum("beni,bend->beid", dup, k_rows[:, None] * lr2 * (pw > 0))
    return torch.cat([g0, g2], dim=2), g1


def test_pool_raw_grad_matches_dense_oracle_and_second_order():
    rows, w02, w1, router, cfg = _setup(seed=1)
    g = torch.Generator().manual_seed(7)
    v_rows = torch.randn(rows.shape, generator=g)
    lr_rows = torch.rand(rows.shape[0], rows.shape[1], 3, generator=g) * 0.1
    for t in (rows, v_rows, lr_rows, w02, w1, router):
        t.requires_grad_(True)
    routing = fw.route_rows(rows, router, None, cfg)
    g02, g1 = fw.pool_raw_grad(rows, v_rows, lr_rows, w02, w1, routing)
    r02, r1 = _dense_raw_grad(rows, v_rows, lr_rows, w02, w1, router, 2)
    torch.testing.assert_close(g02, r02, atol=1e-4, rtol=1e-3)
    torch.testing.assert_close(g1, r1, atol=1e-4, rtol=1e-3)
    # gradient of the inner gradient (what 'full' backward mode needs)
    c02, c1 = torch.randn_like(g02), torch.randn_like(g1)
    ins = [rows, v_rows, lr_rows, w02, w1, router]
    got = torch.autograd.grad([g02, g1], ins, [c02, c1])
    want = torch.autograd.grad([r02, r1], ins, [c02, c1])
    for a, b in zip(got, want):
        torch.testing.assert_close(a, b, atol=2e-4, rtol=2e-3)


def test_apply_update_preserves_row_norms_and_momentum():
    bsz, e, inter, d = 2, 3, 8, 8
    w0 = torch.randn(e, inter, d); w1 = torch.randn(e, d, inter); w2 = torch.randn(e, inter, d)
    st = fw.init_pool_state(w0, w1, w2, bsz, True, torch.float32)
    a02 = torch.randn_like(st.m02); a1 = torch.randn_like(st.m1)
    m = torch.full((bsz, 1, 1, 1), 0.5)
    new = fw.apply_pool_update(a02, a1, st, m, 1.0, True, compute_dtype=torch.float32)
    torch.testing.assert_close(new.m02.norm(dim=3), st.m02.norm(dim=3), atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(new.z02, a02)            # zero initial momentum: Z <- A
    new2 = fw.apply_pool_update(a02, a1, new, m, 1.0, True, compute_dtype=torch.float32)
    torch.testing.assert_close(new2.z02, a02 + 0.5 * a02)


def test_newton_schulz_orthogonalises():
    g = torch.randn(3, 16, 24)
    x = ops.newton_schulz(g)
    s = torch.linalg.svdvals(x.float())
    assert s.max() < 1.3 and s.min() > 0.5


def test_router_types_and_small_ops_on_cpu():
    """The portable statements behind the fused kernels: normalised router types, residual add + norm, embedding."""
    torch.manual_seed(3)
    rows = torch.randn(2, 50, 16)
    router = torch.randn(8, 16)
    bias = torch.randn(8) * 0.01
    for rtype in ("softmax", "norm_softmax", "norm_relu"):
        idx, w, psum = ops.route_topk(rows, router, bias, 2, 0.5, False, True, rtype, 0.0, 1e-6)
        sel, probs = ref.route_scores(rows @ router.t(), rtype, 0.0, 1e-6)
        assert torch.equal(idx, (sel + bias).topk(2, -1).indices)
        picked = probs.gather(-1, idx)
        torch.testing.assert_close(w, (picked / picked.sum(-1, keepdim=True) * 0.5).view(-1, 2))
        torch.testing.assert_close(psum, probs.sum(1))
        torch.testing.assert_close(psum.sum(-1), torch.full((2,), 50.0))      # every variant yields a distribution
    x, delta, wgt = torch.randn(7, 16), torch.randn(7, 16), torch.rand(16) + 0.5
    s, y = ops.add_rms_norm(x, delta, wgt, 1e-6)
    torch.testing.assert_close(s, x + delta)
    torch.testing.assert_close(y, ops.rms_norm(x + delta, wgt, 1e-6))
    from uttt_b200.models.common import TokenEmbedding
    emb = TokenEmbedding(11, 8, padding_idx=3)
    ids = torch.tensor([[1, 3, 3, 10], [0, 1, 1, 1]])
    out = emb(ids)
    assert torch.equal(out, emb.weight[ids])
    out.sum().backward()
    assert float(emb.weight.grad[3].abs().sum()) == 0.0 and float(emb.weight.grad[1].sum()) == 4 * 8


def test_pool_statistics_are_reported_on_their_interval(monkeypatch):
    """The `moe/*` statistics of the reference trainer: usage, dead experts, entropy, selected-weight percentiles."""
    import math
    import torch
    from uttt_b200.config import named_config
    from uttt_b200.models import build_model
    from uttt_b200.models import moe_stats as ms
    cfg = named_config("tiny-uttt-moe", memory_num_active_experts=2)
    model = build_model(cfg).train()
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(0))
    monkeypatch.setenv("UTTT_MOE_STATS_INTERVAL", "5")
    monkeypatch.setenv("FLAME_TRAIN_STEP", "3")
    assert "moe" not in model(input_ids=ids, labels=ids).moe_stats
    monkeypatch.setenv("FLAME_TRAIN_STEP", "10")
    out = model(input_ids=ids, labels=ids)
    moe = out.moe_stats["moe"]
    e = cfg.memory_num_experts
    for prefix in ("apply", "update"):
        assert 0.0 <= float(moe[f"{prefix}_freq_min"]) <= 1.0 / e <= float(moe[f"{prefix}_freq_max"]) <= 1.0
        assert 0.0 < float(moe[f"{prefix}_entropy_ratio"]) <= 1.0 + 1e-6
        assert 0.0 <= float(moe[f"{prefix}_router_entropy"]) <= math.log(e) + 1e-5
        lo, p50, p95, hi = (float(moe[f"{prefix}_selected_weight_{k}"]) for k in ("min", "p50", "p95", "max"))
        assert 0.0 <= lo <= p50 <= p95 <= hi <= 1.0
    out.loss.backward()                                            # the recompute pass must not collect again
    assert all(layer.route_stats is None for layer in model.model.layers)
    # usage statistics from known counts: one dead expert out of four
    counts = torch.tensor([[[10.0, 10.0, 20.0, 0.0]]])
    u = ms.expert_usage_stats(counts, 4, "x")
    assert float(u["x_dead_frac_0p25"]) == 0.25 and float(u["x_freq_max_over_uniform"]) == 2.0
    assert float(ms.expert_usage_stats(torch.zeros(1, 1, 4), 4, "x")["x_freq_max"]) == 0.0
