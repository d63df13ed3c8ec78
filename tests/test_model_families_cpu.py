"""Every registered language-model family builds, trains one step on CPU, and honours its contract."""
import pytest
import torch

from uttt_b200.config import config_from_dict, load_config, named_config
from uttt_b200.models import build_model, registered_model_types
from uttt_b200.models.generation import generate

BASE = dict(hidden_size=64, num_hidden_layers=2, num_heads=4, vocab_size=256, chunk_size=32, window_size=32,
            max_position_embeddings=128, use_memory_block=True, fw_num_heads=2, base_lr=0.001, per_head_lr=True,
            memory_kv_mode="reuse_kv", memory_kv_feature="x_attn_in", memory_qkv_silu=True, memory_qk_norm=True,
            memory_qk_rescale=True, learnable_ttt_scale=True, same_rope=True, use_momentum=True, use_moun=True,
            enable_attention_memory_output_proj=True, rope_theta=10000.0, w0_w2_low_rank=0)


def _ids(seed=0, b=2, s=96):
    return torch.randint(0, 256, (b, s), generator=torch.Generator().manual_seed(seed))


@pytest.mark.parametrize("model_type,extra", [
    ("uttt_dense", dict(uttt_dense_r=2)),
    ("uttt_dense", dict(uttt_dense_r=2, w0_w2_low_rank=4, uttt_agg_reduce="sum", uttt_master_renorm=True)),
    ("ttt_dense", dict(fw_inter_multi=2)),
    ("lact_swiglu", dict(num_lact_heads=2, inter_multi=2, lact_chunk_size=32)),
    ("ttt_moe_lb", dict(fw_inter_multi=2, memory_num_experts=4, memory_num_active_experts=2,
                        memory_lb_mode="loss_free", memory_loss_free_update_rate=1e-2)),
    ("ttt_moe_no_lb", dict(fw_inter_multi=2, memory_num_experts=4, memory_lb_loss_alpha=0.01)),
    ("uttt_moe", dict(fw_inter_multi=2, memory_num_experts=4, memory_num_active_experts=2,
                      memory_update_aggregate_write=False, memory_update_backward_mode="stop_state")),
    ("uttt_moe", dict(fw_inter_multi=2, memory_num_experts=4, memory_update_aggregate_write=True,
                      memory_aggregate_momentum_mode="pool_mean", memory_update_backward_mode="first_order_state",
                      memory_write_layers="last", memory_router_type="norm_softmax",
                      memory_router_combine_mode="topk_renorm", memory_router_share_mode="share_all")),
])
def test_family_forward_backward(model_type, extra):
    torch.manual_seed(0)
    cfg = config_from_dict(dict(BASE, model_type=model_type, **extra))
    model = build_model(cfg)
    ids = _ids()
    out = model(input_ids=ids, labels=ids)
    assert torch.isfinite(out.loss)
    out.loss.backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    if getattr(cfg, "memory_update_backward_mode", "full") in ("stop_state", "first_order_state"):
        # a detached state leaves the write-only heads (learning rates, momentum gate) without gradient
        missing = [n for n in missing if "to_lr" not in n and "momentum_proj" not in n]
    assert not missing, missing
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)


@pytest.mark.parametrize("mt", ["transformer", "deltanet_swa", "gated_deltanet_swa", "kda_swa", "mamba2_swa", "mom_swa"])
def test_baseline_families(mt):
    torch.manual_seed(0)
    cfg = config_from_dict(dict(model_type=mt, hidden_size=64, num_hidden_layers=2, num_heads=4, vocab_size=128,
                                window_size=16, mixer_head_dim=16, rope_theta=10000.0))
    m = build_model(cfg)
    ids = torch.randint(0, 128, (2, 40))
    out = m(input_ids=ids, labels=ids)
    out.loss.backward()
    assert torch.isfinite(out.loss) and all(p.grad is not None for p in m.parameters())
    # causality: a later token does not change earlier positions
    m.eval()
    ids2 = ids.clone()
    ids2[:, 30] = (ids2[:, 30] + 1) % 128
    with torch.no_grad():
        h1, h2 = m(input_ids=ids).hidden_states, m(input_ids=ids2).hidden_states
    torch.testing.assert_close(h1[:, :30], h2[:, :30], atol=1e-5, rtol=1e-5)


def test_registry_covers_reference_model_types():
    have = set(registered_model_types())
    for t in ("uttt_moe", "uttt_dense", "ttt_moe_lb", "ttt_moe_no_lb", "ttt_dense", "lact_swiglu", "transformer",
              "deltanet_swa", "gated_deltanet_swa", "kda_swa", "mamba2_swa", "mom_swa"):
        assert t in have


def test_cross_layer_cut_forward_equals_full_and_cuts_routes():
    torch.manual_seed(0)
    common = dict(BASE, model_type="uttt_moe", fw_inter_multi=2, memory_num_experts=4, memory_num_active_experts=1,
                  memory_update_aggregate_write=True, memory_aggregate_momentum_mode="pool_mean",
                  memory_router_share_mode="per_layer", memory_lb_loss_alpha=0.0)
    full = build_model(config_from_dict(dict(common, memory_update_backward_mode="full")))
    cut = build_model(config_from_dict(dict(common, memory_update_backward_mode="cross_layer_cut")))
    cut.load_state_dict(full.state_dict())
    ids = _ids(1)
    lf = full(input_ids=ids, labels=ids).loss
    lc = cut(input_ids=ids, labels=ids).loss
    torch.testing.assert_close(lf, lc, atol=1e-5, rtol=1e-5)
    lf.backward()
    lc.backward()
    # the last layer's parameters only see their own stream in both modes early on, but the pool
    # parameters receive different gradients once the cross-layer routes are cut
    gf = full.model.layers[0].to_lr.weight.grad
    gc = cut.model.layers[0].to_lr.weight.grad
    assert torch.isfinite(gc).all() and gc.abs().sum() > 0
    assert (gf - gc).abs().max() > 0
    # eval / no-grad forwards run the unchanged full path
    cut.eval()
    with torch.no_grad():
        torch.testing.assert_close(cut(input_ids=ids, labels=ids).loss, lf.detach(), atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("over", [
    dict(),
    # write sources other than the attention's own k / v of the same layer: the cache keeps what they read
    dict(memory_v_gap=1),
    dict(memory_kv_mode="to_kv", memory_kv_proj="ttt_kv_proj", memory_kv_feature="x_memory_in",
         residual_style="sequential"),
], ids=["default sources", "values from the next layer", "own projections of the memory input"])
def test_cached_generation_matches_one_shot_forward(over):
    torch.manual_seed(0)
    cfg = config_from_dict(dict(BASE, model_type="uttt_moe", fw_inter_multi=2, memory_num_experts=4,
                                memory_update_aggregate_write=True, memory_aggregate_momentum_mode="pool_mean",
                                memory_update_backward_mode="full", **over))
    model = build_model(cfg).eval()
    ids = _ids(2, b=1, s=80)
    with torch.no_grad():
        ref = model(input_ids=ids).logits
        out = model(input_ids=ids[:, :50], use_cache=True)
        parts = [out.logits]
        cache = out.past_key_values
        for t in range(50, 80):
            out = model(input_ids=ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            cache = out.past_key_values
            parts.append(out.logits)
    got = torch.cat(parts, dim=1)
    torch.testing.assert_close(got, ref, atol=2e-4, rtol=2e-4)
    toks = generate(model, ids[:, :10], max_new_tokens=5)
    assert toks.shape == (1, 15)


def test_loss_free_bias_moves_against_overloaded_experts():
    torch.manual_seed(0)
    cfg = config_from_dict(dict(BASE, model_type="uttt_moe", fw_inter_multi=2, memory_num_experts=4,
                                memory_update_aggregate_write=True, memory_aggregate_momentum_mode="pool_mean",
                                memory_lb_mode="loss_free", memory_lb_scope="pool", memory_loss_free_update_rate=0.1))
    model = build_model(cfg).train()
    ids = _ids(3)
    model(input_ids=ids, labels=ids)
    counts = model.model.memory_loss_free_pending_counts.clone()
    assert counts.sum() > 0
    model(input_ids=ids, labels=ids)          # the update happens at the start of the next forward
    bias = model.model.memory_loss_free_bias
    assert int(model.model.memory_loss_free_num_updates) == 1
    assert abs(float(bias.mean())) < 1e-6
    over = counts > counts.mean()
    assert bool((bias[over] < 0).all()) and bool((bias[counts < counts.mean()] > 0).all())


def test_lact_accepts_and_writes_the_reference_key_layout():
    """The LaCT baseline's parameters under the reference's names: everything of a layer below ``attn`` with a fused
    ``qkv`` projection (lact/lact_model/layer_lact_swiglu.py).  Loading that layout and writing it back is lossless."""
    cfg = load_config("configs/lm/main/124M/lact.json")
    d = cfg.to_dict()
    d.update(hidden_size=64, num_hidden_layers=2, num_heads=4, num_attn_heads=4, vocab_size=256, num_lact_heads=2,
             w0_w2_low_rank=4, window_size=32, lact_chunk_size=32, chunk_size=32, max_position_embeddings=128)
    torch.manual_seed(0)
    a, b = build_model(config_from_dict(d)), build_model(config_from_dict(d))
    theirs = a.reference_state_dict()
    for key, shape in (("model.layers.0.attn.qkv.weight", (192, 64)), ("model.layers.1.attn.o_proj.weight", (64, 64)),
                       ("model.layers.0.attn.lr_proj.weight", None), ("model.layers.0.attn.w0.w_left", (2, 32, 4)),
                       ("model.layers.0.attn.w1", (2, 32, 32)), ("model.layers.0.attn.ttt_norm.weight", None),
                       ("model.layers.0.attn.momentum_proj.0.bias", None), ("model.layers.0.attn.qk_scale", None),
                       ("model.layers.0.mlp.gate_proj.weight", None), ("lm_head.weight", (256, 64))):
        assert key in theirs, key
        assert shape is None or tuple(theirs[key].shape) == shape, key
    assert not any(".memory." in k or ".to_lr." in k or "q_proj" in k for k in theirs)
    assert len(theirs) == len(a.state_dict()) - 4                      # q, k, v fused per layer
    res = b.load_state_dict(theirs, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    for (k, va), vb in zip(a.state_dict().items(), b.state_dict().values()):
        assert torch.equal(va, vb), k
    ids = torch.randint(0, 256, (1, 64))
    with torch.no_grad():
        torch.testing.assert_close(a(input_ids=ids, labels=ids).loss, b(input_ids=ids, labels=ids).loss)
