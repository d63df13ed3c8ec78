"""View-synthesis half on CPU: model contract, schedules, data tools, checkpoint lifecycle, trainer step."""
import os

import pytest
import torch

from uttt_b200.nvs import checkpoint as ck
from uttt_b200.nvs.data import (NVSDataset, ResumableDistributedSampler, SyntheticScenes, check_manifest,
                                make_toy_dataset)
from uttt_b200.nvs.metrics import bootstrap_ci, psnr, ssim
from uttt_b200.nvs.model import LVSMModel
from uttt_b200.nvs.schedule import inputs_then_targets_config, parallel_ttt_config
from uttt_b200.nvs.trainer import NVSTrainer, apply_overrides, check_batch_arithmetic
from uttt_b200.ops import reference as ref


def _cfg(block="uttt_nvs.models.uttt_moe_block.MemoryModel", **params):
    p = dict(attn_head_dim=32, fw_head_dim=32, inter_multi=2, fw_inter_multi=1, use_muon=False, num_experts=4,
             num_active_experts=2, l2_norm=True, pool_mode="shared", router_share_mode="share_all",
             aggregate_write=True, load_balancing_loss_alpha=1e-5)
    p.update(params)
    if "only" in params:                     # a family with its own parameter set (strict signatures)
        p = dict(params["only"])
    return {"exp_name": "t", "model": {"image_size": 32, "patch_size": 8, "dim": 64, "layers": 2,
                                       "block_config": {"type": block, "params": p}},
            "training": {"batch_size_per_gpu": 2, "total_batch_size": 2, "num_views": 4, "lr": 1e-3, "warmup": 0,
                         "max_fwdbwd_passes": 4, "checkpoint_every": 2, "print_every": 100, "dataset": "synthetic"}}


def _batch(b=2, v=4):
    return next(SyntheticScenes(b, v, 32, pin=False))


@pytest.mark.parametrize("block,params", [
    ("uttt_nvs.models.uttt_moe_block.MemoryModel", {}),
    ("uttt_nvs.models.uttt_moe_block.MemoryModel", dict(pool_mode="per_block", aggregate_write=False,
                                                         router_share_mode="per_layer", use_muon=True)),
    ("uttt_nvs.models.uttt_moe_block.MemoryModel", dict(aggregate_write=False)),
    ("uttt_nvs.models.uttt_dense_block.MemoryModel", {}),
    ("uttt_nvs.models.uttt_dense_partitioned.MemoryModel", dict(num_shared_pools=2, fw_inter_multi=2)),
    ("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", dict(num_shared_pools=2)),
    ("uttt_nvs.models.ttt_dense_block.MemoryModel", dict(only=dict(attn_head_dim=32, fw_head_dim=16, inter_multi=2,
                                                                 fw_inter_multi=2, l2_norm=False, use_muon=True))),
    ("uttt_nvs.models.uttt_dense_block.MemoryModel", dict(aggregate_write=False, v_gap=1)),
    ("uttt_nvs.models.transformer_block.MemoryModel", dict(only=dict(attn_head_dim=32, inter_multi=2,
                                                                   transformer_version="v0", vi_rms_norm=True))),
    ("uttt_nvs.models.transformer_block.MemoryModel", dict(only=dict(attn_head_dim=32, transformer_version="v3", v_gap=1,
                                                                   to_kv_mode="per_layer", pre_vi_source="xi_out"))),
    ("uttt_nvs.models.transformer_block.MemoryModel", dict(only=dict(attn_head_dim=32, transformer_version="v1", bias=True,
                                                                   use_separate_last_to_kv=True))),
    ("uttt_nvs.models.deltanet_block.MemoryModel", dict(only=dict(attn_head_dim=32, fw_num_heads=2, inter_multi=2,
                                                                repeat_function="repeat", use_short_conv=False,
                                                                use_output_gate=False))),
    ("uttt_nvs.models.deltanet_block.MemoryModel", dict(only=dict(attn_head_dim=32, fw_num_heads=2, expand_v=2.0,
                                                                qk_activation="elu", qk_norm="sum", use_muon=True,
                                                                allow_neg_eigval=True, repeat_function="linear"))),
    ("uttt_nvs.models.gated_deltanet_block.MemoryModel", dict(only=dict(attn_head_dim=32, fw_num_heads=2, expand_v=2.0,
                                                                      repeat_function="repeat", noise_repeat=2))),
])
def test_block_families_train(block, params):
    torch.manual_seed(0)
    model = LVSMModel(_cfg(block, **params))
    out = model(_batch())
    loss = out["loss_metrics"]["loss"]
    assert torch.isfinite(loss) and out["rendering"].shape == (2, 3, 3, 32, 32)
    loss.backward()
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name


def test_state_dict_layout_and_aggregate_differs_from_chained():
    torch.manual_seed(0)
    agg = LVSMModel(_cfg())
    keys = set(agg.state_dict())
    for k in ("image_tokenizer.1.weight", "transformer_input_layernorm.weight", "transformer_blocks.pool_w0",
              "transformer_blocks.shared_router_proj_weights", "transformer_blocks.blocks.0.ln_attn.weight",
              "transformer_blocks.blocks.0.self_attention.to_qkv.weight",
              "transformer_blocks.blocks.1.memory.k_input_proj.0.weight", "transformer_blocks.blocks.0.memory.to_lr.weight",
              "transformer_blocks.blocks.0.mlp.gate.weight", "image_token_decoder.0.weight", "image_token_decoder.1.weight"):
        assert k in keys, k
    chained = LVSMModel(_cfg(aggregate_write=False))
    chained.load_state_dict(agg.state_dict())
    b = _batch()
    with torch.no_grad():
        a, c = agg(b)["rendering"], chained(b)["rendering"]
    assert (a - c).abs().max() > 1e-7                 # one write from a shared snapshot != writes in turn
    one = LVSMModel(dict(_cfg(), model=dict(_cfg()["model"], layers=1)))
    one_c = LVSMModel(dict(_cfg(aggregate_write=False), model=dict(_cfg()["model"], layers=1)))
    one_c.load_state_dict(one.state_dict())
    with torch.no_grad():
        torch.testing.assert_close(one(b)["rendering"], one_c(b)["rendering"])   # equal with a single layer


def test_inputs_then_targets_layout():
    cfg = _cfg()
    cfg["model"].update(view_layout="inputs_then_targets", num_input_views=3)
    model = LVSMModel(cfg)
    out = model(_batch(v=5))
    assert out["rendering"].shape[1] == 2
    sched = inputs_then_targets_config(4, 2, 16)
    assert [c.update for c in sched] == [True] * 4 + [False] * 2
    par = parallel_ttt_config(16, 16, 96)
    assert [c.update for c in par] == [True, False] * 3


def test_plucker_rays_are_unit_and_orthogonal_moment():
    b = _batch()
    o, d = ref.plucker_rays(b["fxfycxcy"], b["c2w"], 32, 32)
    torch.testing.assert_close(d.norm(dim=2), torch.ones_like(d[:, :, 0]), atol=1e-5, rtol=1e-5)
    m = torch.cross(o, d, dim=2)
    assert (m * d).sum(2).abs().max() < 1e-4          # o x d is perpendicular to d
    # the central ray of a camera on the sphere looks at the origin
    centre = d[..., 16, 16] + d[..., 15, 15]
    eye = b["c2w"][..., :3, 3]
    cos = torch.nn.functional.cosine_similarity(centre, -eye, dim=-1)
    assert cos.min() > 0.999
    tok = ref.plucker_embed(b["image"], b["fxfycxcy"], b["c2w"], torch.tensor([False, True, False, True]), 8)
    assert tok.shape == (2, 4, 16, 8 * 8 * 12)
    assert tok[:, 1].reshape(2, 16, 64, 12)[..., 9:].abs().max() == 0     # pose-only views carry zero RGB


def test_toy_dataset_is_deterministic_and_right_handed(tmp_path):
    m1 = make_toy_dataset(str(tmp_path / "a"), 2, 6, 32, seed=3)
    m2 = make_toy_dataset(str(tmp_path / "b"), 2, 6, 32, seed=3)
    assert check_manifest(m1) == []
    d1, d2 = NVSDataset(m1, 4, 32), NVSDataset(m2, 4, 32)
    torch.testing.assert_close(d1[0]["image"], d2[0]["image"])
    rot = d1[1]["c2w"][:, :3, :3]
    torch.testing.assert_close(torch.det(rot), torch.ones(4), atol=1e-4, rtol=1e-4)
    with open(m1, "a") as fh:
        fh.write(str(tmp_path / "missing.json") + "\n")
    assert check_manifest(m1)


def test_sampler_resume_skips_consumed_samples():
    ds = list(range(40))
    s = ResumableDistributedSampler(ds, num_replicas=2, rank=0, shuffle=True, seed=0)
    s.set_epoch(3)
    full = list(iter(s))
    s.set_resume_offset(7)
    assert list(iter(s)) == full[7:]
    assert list(iter(s)) == full                      # the skip applies once
    with pytest.raises(ValueError):
        s.set_resume_offset(len(full))
        list(iter(s))


class _Obj:
    def __init__(self):
        self.v = {"a": 1}

    def state_dict(self):
        return self.v

    def load_state_dict(self, sd):
        self.v = sd


def test_checkpoint_lifecycle(tmp_path, monkeypatch):
    model = torch.nn.Linear(3, 3)
    opt, sch = _Obj(), _Obj()
    out = str(tmp_path)
    ck.checkpoint_job(out, model, opt, sch, 10, 5)
    ck.checkpoint_job(out, model, opt, sch, 200, 100)
    assert [os.path.basename(p) for p in ck.find_checkpoints(out)] == ["ckpt_0000000000000010.pt",
                                                                       "ckpt_0000000000000200.pt"]
    # a failed save leaves the previous checkpoints intact and no temporary file behind
    real_save = torch.save
    def boom(*a, **k):
        raise OSError("disk full")
    monkeypatch.setattr(torch, "save", boom)
    with pytest.raises(OSError):
        ck.checkpoint_job(out, model, opt, sch, 300, 150)
    monkeypatch.setattr(torch, "save", real_save)
    assert len(ck.find_checkpoints(out)) == 2 and not [f for f in os.listdir(out) if f.endswith(".tmp")]
    # corrupt newest -> falls back to the older one
    with open(ck.find_checkpoints(out)[-1], "wb") as fh:
        fh.write(b"garbage")
    _, _, step, upd = ck.resume_job(out, torch.nn.Linear(3, 3), _Obj(), _Obj())
    assert (step, upd) == (10, 5)
    # reset keeps weights, zeroes counters
    m2 = torch.nn.Linear(3, 3)
    _, _, step, upd = ck.resume_job(ck.find_checkpoints(out)[0], m2, _Obj(), _Obj(), reset_training_state=True)
    assert (step, upd) == (0, 0)
    torch.testing.assert_close(m2.weight, model.weight)
    # retention, missing path, all corrupt
    ck.delete_previous_job(out, 200, 1)
    assert len(ck.find_checkpoints(out)) == 1
    with pytest.raises(FileNotFoundError):
        ck.resume_job(str(tmp_path / "nope.pt"), model, opt, sch)
    with open(ck.find_checkpoints(out)[0], "wb") as fh:
        fh.write(b"x")
    with pytest.raises(RuntimeError):
        ck.resume_job(out, model, opt, sch)
    assert ck.select_resume_path(out, "explicit.pt", "cfg.pt") == out
    assert ck.select_resume_path(str(tmp_path / "empty"), "explicit.pt", "cfg.pt") == "explicit.pt"


def test_overrides_and_batch_guard():
    cfg = apply_overrides(_cfg(), [["block.num_experts", "8"], ["training.lr", "3e-4"], ["exp_name", "abc"]])
    assert cfg["model"]["block_config"]["params"]["num_experts"] == 8 and cfg["training"]["lr"] == 3e-4
    assert cfg["exp_name"] == "abc"
    cfg["training"]["total_batch_size"] = 16
    with pytest.raises(ValueError):
        check_batch_arithmetic(cfg, 1)


def test_trainer_runs_saves_and_resumes(tmp_path):
    cfg = _cfg()
    cfg["training"]["out_dir"] = str(tmp_path)
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    summary = t.fit()
    assert t.fwdbwd_step == 4 and summary["avg_step_time_s"] > 0
    assert len(ck.find_checkpoints(t.out_dir)) == 2           # passes 2 and 4; the last three are kept by default
    t2 = NVSTrainer(cfg, device=torch.device("cpu"))
    assert t2.fwdbwd_step == 4 and t2.update_step == 4
    for (n1, p1), (n2, p2) in zip(t.model.named_parameters(), t2.model.named_parameters()):
        torch.testing.assert_close(p1, p2, msg=n1)


def test_grad_accumulation_keeps_every_micro_batch(tmp_path):
    """Two passes of b scenes with grad_accum_steps=2 give the same update as one pass of 2b scenes."""
    big = _batch(b=4)

    def run(accum):
        cfg = _cfg(block="uttt_nvs.models.transformer_block.MemoryModel", only=dict(attn_head_dim=32, inter_multi=2, transformer_version="v0"))
        tr = cfg["training"]
        tr.update(out_dir=str(tmp_path / f"a{accum}"), grad_accum_steps=accum, batch_size_per_gpu=4 // accum,
                  total_batch_size=4, grad_clip_norm=0.0, weight_decay=0.0)
        t = NVSTrainer(cfg, device=torch.device("cpu"))
        per = 4 // accum
        for i in range(accum):
            t.train_pass({k: v[i * per:(i + 1) * per] for k, v in big.items() if torch.is_tensor(v)})
        assert t.update_step == 1
        return {n: p.detach().clone() for n, p in t.model.named_parameters()}

    one, two = run(1), run(2)
    moved = 0
    for n in one:
        torch.testing.assert_close(two[n], one[n], rtol=1e-4, atol=2e-5, msg=n)
    # dropping the last micro-batch changes the update by far more than the tolerance above
    ref0 = {n: p.detach().clone() for n, p in NVSTrainer(
        {**_cfg(block="uttt_nvs.models.transformer_block.MemoryModel", only=dict(attn_head_dim=32, inter_multi=2, transformer_version="v0")),
         "training": {**_cfg()["training"], "out_dir": str(tmp_path / "z")}},
        device=torch.device("cpu")).model.named_parameters()}
    assert any((one[n] - ref0[n]).abs().max() > 1e-4 for n in one)


def test_metrics():
    a = torch.rand(3, 3, 32, 32)
    assert float(ssim(a, a).min()) > 0.999
    assert float(psnr(a, a).min()) > 90
    noisy = (a + 0.1 * torch.randn_like(a)).clamp(0, 1)
    assert float(ssim(a, noisy).mean()) < 0.99
    ci = bootstrap_ci([20.0, 21.0, 22.0, 23.0], resamples=2000)
    assert ci["ci_low"] <= ci["mean"] <= ci["ci_high"]


def test_debug_helpers_and_trace_ranges():
    from uttt_b200.nvs.debug import RouterTrace, log_status, sketch_tensor
    from uttt_b200.utils import trace
    t = torch.tensor([[1.0, 2.0], [float("nan"), 4.0]])
    s = sketch_tensor(t, "x")
    assert s["non_finite"] == 1 and s["shape"] == [2, 2] and abs(s["max"] - 4.0) < 1e-6
    lines = []
    rows = log_status({"a": torch.ones(3), "b": torch.zeros(0)}, lines.append)
    assert len(rows) == 2 and len(lines) == 1 and lines[0].startswith("a")
    tr = RouterTrace()
    tr(0, "read", torch.tensor([[3.0, 1.0]]), torch.tensor([[2.0, 2.0]]))
    assert tr.summary()["freq_max"] == 0.75
    trace.enable(True)
    try:
        with trace.trace_range("unit-test"):
            pass
    finally:
        trace.enable(False)
    assert not trace.enabled()


def test_checkpoint_grouping_and_sweep_do_not_change_the_numbers():
    """`apply_ckpt_group` and `update_ckpt_sweep` only change where activations are recomputed: same loss and the
    same gradients as the default schedule; invalid group sizes are rejected; master offload is a no-op on CPU."""
    batch = _batch()
    results = []
    for params in (dict(), dict(apply_ckpt_group=2), dict(update_ckpt_sweep=True),
                   dict(apply_ckpt_group=2, update_ckpt_sweep=True, offload_master_states=True)):
        torch.manual_seed(0)
        model = LVSMModel(_cfg(**params))
        out = model(batch)
        out["loss_metrics"]["loss"].backward()
        results.append((float(out["loss_metrics"]["loss"]),
                        {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}))
    for loss, grads in results[1:]:
        assert loss == pytest.approx(results[0][0], rel=1e-6)
        for n, g in results[0][1].items():
            torch.testing.assert_close(grads[n], g, rtol=1e-4, atol=1e-6, msg=n)
    with pytest.raises(ValueError):
        LVSMModel(_cfg(apply_ckpt_group=3))
    with pytest.raises(ValueError):
        LVSMModel(_cfg(aggregate_write=False, offload_master_states=True))
    with pytest.raises(ValueError, match="shared_expert_per_layer"):
        LVSMModel(_cfg(use_shared_expert=True))               # aggregated write + one expert for the whole stack


def test_shared_expert_raw_gradient_is_the_squared_error_gradient():
    """The always-on expert's raw update equals autograd's gradient of 1/2 |f(k) - v|^2, each matrix scaled by its
    learning rate averaged over the sequence (uttt_nvs/models/uttt_moe_block.py:425-462)."""
    from uttt_b200.nvs.blocks import FastWeightMemory
    torch.manual_seed(0)
    b, t, d, inter = 2, 24, 16, 32
    k, v = torch.randn(b, t, d), torch.randn(b, t, d)
    lr = torch.rand(b, t, 3)
    se = tuple(torch.randn(b, 1, *shape, requires_grad=True) for shape in ((inter, d), (d, inter), (inter, d)))
    d0, d1, d2 = FastWeightMemory.shared_expert_grad(k, v, lr, tuple(w.detach() for w in se))
    out = FastWeightMemory.shared_expert_ffn(k, se)
    g0, g1, g2 = torch.autograd.grad(0.5 * (out - v).pow(2).sum(), se)
    mean = lr.mean(dim=1)
    for got, want, i in ((d0, g0, 0), (d1, g1, 1), (d2, g2, 2)):
        torch.testing.assert_close(got, want * mean[:, i].view(b, 1, 1, 1), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("aggregate", [True, False])
def test_view_synthesis_with_per_layer_shared_expert(aggregate):
    """``use_shared_expert`` with one always-on expert per layer: the parameters carry the reference's names, take
    gradients, and the model differs from the one without it."""
    from uttt_b200.nvs.data import SyntheticScenes
    from uttt_b200.nvs.model import LVSMModel
    params = {"attn_head_dim": 16, "fw_head_dim": 16, "inter_multi": 2, "fw_inter_multi": 1, "use_muon": False,
              "num_experts": 4, "num_active_experts": 2, "l2_norm": True, "pool_mode": "shared",
              "router_share_mode": "share_all", "aggregate_write": aggregate, "use_shared_expert": True,
              "shared_expert_per_layer": True}
    cfg = {"model": {"image_size": 16, "patch_size": 8, "dim": 32, "layers": 2,
                     "block_config": {"type": "uttt_nvs.models.uttt_moe_block.MemoryModel", "params": params}},
           "training": {"num_views": 3, "lpips_loss_weight": 0.0}}
    torch.manual_seed(0)
    model = LVSMModel(cfg)
    keys = set(model.state_dict())
    for name in ("w0", "w1", "w2"):
        for layer in range(2):
            assert f"transformer_blocks.shared_expert_{name}_list.{layer}" in keys
    batch = next(SyntheticScenes(2, 3, 16, seed=1, rank=0, pin=False))
    out = model(batch)
    out["loss_metrics"]["loss"].backward()
    for name in ("w0", "w1", "w2"):
        for p in getattr(model.transformer_blocks, f"shared_expert_{name}_list"):
            assert p.grad is not None and float(p.grad.abs().max()) > 0
    # one expert for the whole stack works with chained writes only (an aggregated write has no order of layers)
    params2 = dict(params, shared_expert_per_layer=False)
    cfg2 = {"model": {**cfg["model"], "block_config": {"type": cfg["model"]["block_config"]["type"], "params": params2}},
            "training": cfg["training"]}
    if aggregate:
        with pytest.raises(ValueError, match="shared_expert_per_layer"):
            LVSMModel(cfg2)
    else:
        assert "transformer_blocks.shared_expert_w0" in LVSMModel(cfg2).state_dict()


def test_partitioned_pool_layout_and_rebinding():
    """Flat parameter layout of the depth-partitioned routed stack, both router modes, and the group runners following
    the registered parameters through a conversion that replaces them."""
    base = dict(num_shared_pools=2, num_experts=4, aggregate_write=True)
    per_pool = LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", router_share_mode="share_pool", **base))
    keys = set(per_pool.state_dict())
    for k in ("transformer_blocks.pool_w0_list.0", "transformer_blocks.pool_w2_list.1",
              "transformer_blocks.pool_router_proj_weights_list.1", "transformer_blocks.blocks.1.memory.to_lr.weight"):
        assert k in keys, k
    assert not any(".parts." in k for k in keys) and "transformer_blocks.shared_router_proj_weights" not in keys
    assert per_pool.state_dict()["transformer_blocks.pool_w0_list.0"].shape[1] == 2          # experts per pool
    one_router = LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", **base))    # share_all
    stack = one_router.transformer_blocks
    assert "transformer_blocks.shared_router_proj_weights" in one_router.state_dict()
    assert all(p.shared_router_proj_weights is stack.shared_router_proj_weights for p in stack.parts)
    assert len(list(one_router.parameters())) == len(one_router.state_dict())                  # nothing counted twice
    b = _batch()
    with torch.no_grad():
        before = one_router(b)["rendering"]
    copy_ = LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", **base))
    with torch.device("meta"):
        hollow = LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", **base))
    hollow = hollow.to_empty(device="cpu")                     # new parameter objects everywhere
    hollow.load_state_dict(one_router.state_dict())
    copy_.load_state_dict(one_router.state_dict())
    with torch.no_grad():
        torch.testing.assert_close(copy_(b)["rendering"], before)
        torch.testing.assert_close(hollow(b)["rendering"], before)
    with pytest.raises(NotImplementedError):
        LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", v_gap=1, **base))
    with pytest.raises(ValueError):
        LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", num_shared_pools=2, num_experts=3))


def test_job_overview_rounds_the_pass_budget_to_epochs():
    from uttt_b200.nvs.trainer import job_overview
    o = job_overview(num_gpus=4, num_train_samples=1000, batch_size_per_gpu=8, grad_accum_steps=2,
                     max_fwdbwd_passes=100)
    assert o["num_fwdbwd_passes_per_epoch"] == 31 and o["num_epochs"] == 4 and o["num_fwdbwd_passes"] == 124
    assert o["num_param_updates"] == 62 and o["batch_size_per_param_update"] == 64
    exact = job_overview(4, 1000, 8, 2, 100, round_max_fwdbwd_passes_to_epoch=False)
    assert exact["num_fwdbwd_passes"] == 100 and exact["num_epochs"] == 4 and exact["num_param_updates"] == 50
    assert job_overview(8, 10, 4, 1, 5)["num_fwdbwd_passes_per_epoch"] == 1          # fewer samples than one pass


def test_in_training_evaluation_visuals_metrics_and_warmup(tmp_path):
    """Evaluation after the first pass and every ``eval_every`` passes (24-view synthetic scenes here), visuals every
    ``vis_every`` passes, a metrics line per logged pass, and the squared-error-only warm-up."""
    import json
    cfg = _cfg()
    cfg["training"].update(out_dir=str(tmp_path), max_fwdbwd_passes=4, eval_every=3, vis_every=2, eval_num_views=5,
                           checkpoint_every=100, l2_warmup_steps=2, print_every=1)
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    warm = []
    real_pass = t._forward_backward
    t._forward_backward = lambda b: (warm.append(t.model._l2_only), real_pass(b))[1]
    t.fit()
    assert warm == [True, True, False, False]
    made = sorted(os.listdir(t.out_dir))
    assert {"eval_00000001", "eval_00000003", "iter_00000002", "iter_00000004", "metrics.jsonl"} <= set(made)
    files = sorted(os.listdir(os.path.join(t.out_dir, "eval_00000003")))
    assert files[0].startswith("input_") and files[1].startswith("supervision_") and files[2] == "uids.txt"
    from PIL import Image
    w, h = Image.open(os.path.join(t.out_dir, "eval_00000003", files[1])).size
    assert (w, h) == (4 * 2 * 32, 2 * 32)                     # 4 scored views x (target | rendering), 2 scenes
    lines = [json.loads(ln) for ln in open(os.path.join(t.out_dir, "metrics.jsonl"))]
    train = [ln for ln in lines if "train/loss" in ln]
    evals = [ln for ln in lines if "eval/loss" in ln]
    assert [ln["step"] for ln in train] == [1, 2, 3, 4] and [ln["step"] for ln in evals] == [1, 3]
    assert {"eval/psnr", "eval/moe_freq_max", "eval_loc/psnr_loc_000", "eval_loc/psnr_loc_003"} <= set(evals[0])
    assert t.model.training and not t.model._l2_only
    out = t.model(_batch())
    assert set(out) == {"input", "target", "loss_metrics", "rendering", "op2block2info"}
    assert out["target"].image.shape == (2, 3, 3, 32, 32) and out["input"]["c2w"].shape == (2, 3, 4, 4)


def test_trainer_refuses_what_the_reference_refuses(tmp_path):
    cfg = _cfg()
    cfg["training"]["out_dir"] = str(tmp_path)
    cfg["model"]["act_ckpt"] = True
    with pytest.raises(NotImplementedError, match="act_ckpt"):
        NVSTrainer(cfg, device=torch.device("cpu"))
    cfg["model"]["act_ckpt"] = False
    manifest = make_toy_dataset(str(tmp_path / "toy"), num_scenes=2, num_frames=6, image_size=32, repeat=2)
    cfg["training"].update(dataset="toy", dataset_path=manifest, max_fwdbwd_passes=1, eval_every=1)
    cfg["eval_dataset_path"] = "PATH/TO/eval_manifest.txt"
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    assert t.num_train_samples == 4 and t.overview["num_fwdbwd_passes_per_epoch"] == 2
    assert t.total == 2                                        # one pass asked for, rounded up to the epoch
    with pytest.raises(ValueError, match="eval_dataset_path"):
        t.fit()
    cfg["eval_dataset_path"] = manifest
    cfg["training"].update(eval_num_views=6, out_dir=str(tmp_path / "second"))
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    t.fit()
    assert os.path.isdir(os.path.join(t.out_dir, "eval_00000002")) and t.fwdbwd_step == 2
    small = make_toy_dataset(str(tmp_path / "small"), num_scenes=1, num_frames=6, image_size=32, repeat=1)
    cfg["training"].update(dataset_path=small, out_dir=str(tmp_path / "third"))
    with pytest.raises(ValueError, match="zero complete batches"):   # one entry, two samples per batch
        NVSTrainer(cfg, device=torch.device("cpu")).fit()


def test_learning_rate_schedule_values():
    """Against torch's LambdaLR with the multiplier written out: step k of the optimizer runs at lambda(k)."""
    import math
    from uttt_b200.nvs.trainer import lr_at

    def expected(k, warmup, total, kind, init):
        if warmup > 0 and k < warmup:
            return init + (1 - init) * k / warmup
        if kind == "constant" or total <= warmup:
            return 1.0
        if kind == "linear":
            return max(0.0, (total - k) / max(1, total - warmup))
        return 0.5 * (1 + math.cos(math.pi * min(max((k - warmup) / max(1, total - warmup), 0), 1)))

    for kind in ("cosine", "linear", "constant"):
        for init in (0.0, 0.25):
            p = torch.nn.Parameter(torch.zeros(1))
            opt = torch.optim.SGD([p], lr=2.0)
            sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda k, kind=kind, init=init: expected(k, 5, 20, kind, init))
            for k in range(24):
                assert lr_at(k, 2.0, 5, 20, kind, init) == pytest.approx(opt.param_groups[0]["lr"]), (kind, init, k)
                opt.step()
                sched.step()
    assert lr_at(0, 1.0, 10, 100) == 0.0 and lr_at(10, 1.0, 10, 100) == 1.0 and lr_at(100, 1.0, 10, 100) == pytest.approx(0.0)
    assert lr_at(3, 1.0, 0, 100, "constant") == 1.0
    with pytest.raises(ValueError):
        lr_at(0, 1.0, 1, 10, "step")


def test_resume_from_a_checkpoint_in_the_reference_format(tmp_path):
    """A checkpoint as the reference's trainer writes it: fp32 weights under DDP / compile prefixes, the state of a
    ``torch.optim.AdamW`` with (rank >= 2 | rest) parameter groups, a ``LambdaLR`` state, the two counters."""
    torch.manual_seed(0)
    cfg = _cfg()
    cfg["training"].update(out_dir=str(tmp_path / "run"), max_fwdbwd_passes=8)
    src = LVSMModel(cfg)
    named = list(src.named_parameters())
    opt = torch.optim.AdamW([{"params": [p for _, p in named if p.dim() >= 2], "weight_decay": 0.05},
                             {"params": [p for _, p in named if p.dim() < 2], "weight_decay": 0.0}], lr=1e-3)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda k: 1.0)
    for _ in range(3):
        src(_batch())["loss_metrics"]["loss"].backward()
        opt.step()
        sched.step()
        opt.zero_grad()
    os.makedirs(tmp_path / "theirs")
    path = str(tmp_path / "theirs" / "ckpt_0000000000000003.pt")
    torch.save({"model": {"module._orig_mod." + k: v for k, v in src.state_dict().items()}, "optimizer": opt.state_dict(),
                "lr_scheduler": sched.state_dict(), "fwdbwd_pass_step": 3, "param_update_step": 3}, path)
    t = NVSTrainer(cfg, device=torch.device("cpu"), load=path)
    assert (t.fwdbwd_step, t.update_step, t.schedule.step_count, t.trainer.step_count) == (3, 3, 3, 3)
    ours = t.trainer.optimizer_state_dict()["state"]
    theirs = opt.state_dict()["state"]
    order = [n for n, p in named if p.dim() >= 2] + [n for n, p in named if p.dim() < 2]
    assert set(ours) == set(order)
    for idx, name in enumerate(order):
        torch.testing.assert_close(ours[name]["exp_avg"], theirs[idx]["exp_avg"], msg=name)
        torch.testing.assert_close(ours[name]["exp_avg_sq"], theirs[idx]["exp_avg_sq"], msg=name)
        torch.testing.assert_close(ours[name]["master"], dict(named)[name].detach(), msg=name)     # fp32, not re-rounded
    t.fit(max_passes=1)
    assert t.fwdbwd_step == 4
    # and back: what this trainer writes loads into torch's AdamW / LambdaLR the way the reference's resume does it
    blob = torch.load(t.save(), weights_only=False)
    assert blob["optimizer"]["param_groups"][0]["lr"] > 0 and blob["fwdbwd_pass_step"] == 4
    assert all(v.dtype == torch.float32 for k, v in blob["model"].items() if v.is_floating_point())
    dst = LVSMModel(cfg)
    assert not dst.load_state_dict(blob["model"], strict=True).missing_keys
    named2 = list(dst.named_parameters())
    opt2 = torch.optim.AdamW([{"params": [p for _, p in named2 if p.dim() >= 2], "weight_decay": 0.05},
                              {"params": [p for _, p in named2 if p.dim() < 2], "weight_decay": 0.0}], lr=1e-3)
    sched2 = torch.optim.lr_scheduler.LambdaLR(opt2, lambda k: 1.0)
    opt2.load_state_dict(blob["optimizer"])
    sched2.load_state_dict(blob["lr_scheduler"])
    assert sched2.last_epoch == 4 and opt2.param_groups[1]["weight_decay"] == 0.0
    inner = t.trainer.optimizer_state_dict()["state"]
    for idx, name in enumerate(order):
        st = opt2.state[dict(named2)[name]]
        assert float(st["step"]) == 4.0
        torch.testing.assert_close(st["exp_avg"], inner[name]["exp_avg"], msg=name)
        torch.testing.assert_close(dict(named2)[name].detach(), inner[name]["master"], msg=name)
    # a state that does not fit this model is skipped with a warning; weights and counters still load
    other = _cfg(num_experts=8)
    other["training"].update(out_dir=str(tmp_path / "other"), max_fwdbwd_passes=8)
    bad = torch.load(path, weights_only=False)
    bad["optimizer"]["param_groups"][0]["params"] = bad["optimizer"]["param_groups"][0]["params"][:-1]
    torch.save(bad, str(tmp_path / "theirs" / "ckpt_0000000000000004.pt"))
    t2 = NVSTrainer(cfg | {"training": {**cfg["training"], "out_dir": str(tmp_path / "run2")}}, device=torch.device("cpu"),
                    load=str(tmp_path / "theirs" / "ckpt_0000000000000004.pt"))
    assert t2.fwdbwd_step == 3 and not t2.optimizer.loaded
    # weights from elsewhere with a reset: counters start at zero; the run's own folder later wins over `load`
    cfg3 = cfg | {"training": {**cfg["training"], "out_dir": str(tmp_path / "run3"), "reset_training_state": True}}
    t3 = NVSTrainer(cfg3, device=torch.device("cpu"), load=path)
    assert (t3.fwdbwd_step, t3.update_step) == (0, 0)
    t3.fit(max_passes=2)
    assert NVSTrainer(cfg3, device=torch.device("cpu"), load=path).fwdbwd_step == 2


@pytest.mark.parametrize("block,params", [
    ("uttt_nvs.models.uttt_dense_block.MemoryModel",
     dict(only=dict(attn_head_dim=32, fw_head_dim=16, inter_multi=2, fw_inter_multi=2, l2_norm=True, use_muon=False,
                    aggregate_write=True))),
    ("uttt_nvs.models.ttt_dense_block.MemoryModel",
     dict(only=dict(attn_head_dim=32, fw_head_dim=16, inter_multi=2, fw_inter_multi=1, l2_norm=True, use_muon=True))),
    ("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", dict(num_shared_pools=2, router_share_mode="share_pool")),
    ("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", dict(num_shared_pools=2)),
    ("uttt_nvs.models.transformer_block.MemoryModel", dict(only=dict(attn_head_dim=32, transformer_version="v1"))),
    ("uttt_nvs.models.gated_deltanet_block.MemoryModel",
     dict(only=dict(attn_head_dim=32, fw_num_heads=2, repeat_function="repeat"))),
])
def test_every_stack_trains_through_the_sharded_optimizer_and_resumes(tmp_path, block, params):
    """Flat-buffer optimizer units per block (also where blocks are shared with unregistered runners or a projection
    is registered under two names), every parameter moves, and a resumed trainer holds the same weights."""
    cfg = _cfg(block, **params)
    cfg["training"].update(out_dir=str(tmp_path), max_fwdbwd_passes=3, eval_every=0, checkpoint_every=100)
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    before = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    for _ in range(3):
        assert torch.isfinite(t.train_pass(next(t.data))["loss"])
    assert all((p.detach() - before[n]).abs().max() > 0 for n, p in t.model.named_parameters())
    t.save()
    t2 = NVSTrainer(cfg, device=torch.device("cpu"))
    assert t2.fwdbwd_step == 3
    for (k, a), b in zip(t.model.state_dict().items(), t2.model.state_dict().values()):
        assert torch.equal(a, b), k


def test_one_always_on_expert_for_the_whole_stack():
    """``use_shared_expert`` without ``shared_expert_per_layer`` on a shared pool: a single expert (``shared_expert_w0/1/2``)
    that every layer reads and, with chained writes, updates in turn."""
    base = dict(use_shared_expert=True, aggregate_write=False)
    one = LVSMModel(_cfg(**base))
    keys = set(one.state_dict())
    assert {"transformer_blocks.shared_expert_w0", "transformer_blocks.shared_expert_w1",
            "transformer_blocks.shared_expert_w2"} <= keys and not any("shared_expert_w0_list" in k for k in keys)
    out = one(_batch())
    out["loss_metrics"]["loss"].backward()
    for name in ("shared_expert_w0", "shared_expert_w1", "shared_expert_w2"):
        g = getattr(one.transformer_blocks, name).grad
        assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0
    # with a single layer it is the per-layer expert
    cfg1 = _cfg(**base)
    cfg1["model"]["layers"] = 1
    cfg2 = _cfg(shared_expert_per_layer=True, **base)
    cfg2["model"]["layers"] = 1
    a, b = LVSMModel(cfg1), LVSMModel(cfg2)
    sd = {k.replace("shared_expert_w0", "shared_expert_w0_list.0").replace("shared_expert_w1", "shared_expert_w1_list.0")
          .replace("shared_expert_w2", "shared_expert_w2_list.0"): v for k, v in a.state_dict().items()}
    b.load_state_dict(sd)
    batch = _batch()
    with torch.no_grad():
        torch.testing.assert_close(a(batch)["rendering"], b(batch)["rendering"])
    # with two layers the second layer reads what the first one wrote: not the per-layer result
    c, d = LVSMModel(_cfg(**base)), LVSMModel(_cfg(shared_expert_per_layer=True, **base))
    sd = {}
    for k, v in c.state_dict().items():
        if "shared_expert_w" in k:
            for layer in range(2):
                sd[f"{k}_list.{layer}"] = v
        else:
            sd[k] = v
    d.load_state_dict(sd)
    with torch.no_grad():
        assert (c(batch)["rendering"] - d(batch)["rendering"]).abs().max() > 1e-7
    with pytest.raises(ValueError, match="shared_expert_per_layer"):
        LVSMModel(_cfg(use_shared_expert=True, aggregate_write=True))
    with pytest.raises(NotImplementedError):
        LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", num_shared_pools=2, **base))


def test_overrides_aliases_and_command_line(tmp_path, monkeypatch):
    from uttt_b200.nvs.trainer import apply_overrides, main
    cfg = {"model": {"block_config": [{"params": {"a": 1}}, {"params": {}}]}, "training": {}}
    apply_overrides(cfg, [["block1.num_experts", "8"], ["block0.a", "2"], ["training.lr", "3e-4"],
                          ["training.tags", "['x', 'y']"], ["exp_name", "name"]])
    assert cfg["model"]["block_config"][1]["params"]["num_experts"] == 8 and cfg["model"]["block_config"][0]["params"]["a"] == 2
    assert cfg["training"] == {"lr": 3e-4, "tags": ["x", "y"]} and cfg["exp_name"] == "name"
    import yaml
    run = _cfg()
    run["training"].update(out_dir=str(tmp_path / "from_file"), max_fwdbwd_passes=5, eval_every=2)
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(run))
    monkeypatch.setenv("UTTT_NVS_OUT_DIR", str(tmp_path / "from_env"))          # wins over training.out_dir
    main([str(path), "--debug", "--seed", "7", "-s", "block.num_experts", "2", "-s", "block.num_active_experts", "1"])
    out = tmp_path / "from_env" / "t"
    assert sorted(p for p in os.listdir(out) if p.startswith(("ckpt", "eval"))) == ["ckpt_0000000000000001.pt",
                                                                                  "eval_00000001"]
    assert not (tmp_path / "from_file").exists()
    blob = torch.load(out / "ckpt_0000000000000001.pt", weights_only=False)
    assert blob["model"]["transformer_blocks.pool_w0"].shape[1] == 2


def test_group_after_group_equals_the_layer_interleaved_walk():
    """The partitioned stack runs its groups one after the other over the whole schedule.  With one layer per group it
    must give what per-block pools give, which walk the layers chunk by chunk: same weights, same renderings, same
    gradients."""
    torch.manual_seed(0)
    common = dict(aggregate_write=False, num_experts=2, num_active_experts=1)
    part = LVSMModel(_cfg("uttt_nvs.models.uttt_moe_partitioned.MemoryModel", num_shared_pools=2,
                          router_share_mode="share_pool", **{**common, "num_experts": 4}))
    per_block = LVSMModel(_cfg(pool_mode="per_block", router_share_mode="per_layer", **common))
    rename = {"pool_w0_list": "block_w0_list", "pool_w1_list": "block_w1_list", "pool_w2_list": "block_w2_list",
              "pool_router_proj_weights_list": "router_proj_weights_list"}
    sd = {}
    for k, v in part.state_dict().items():
        for old, new in rename.items():
            k = k.replace(f".{old}.", f".{new}.")
        sd[k] = v
    per_block.load_state_dict(sd)
    batch = _batch()
    out_p, out_b = part(batch), per_block(batch)
    torch.testing.assert_close(out_p["rendering"], out_b["rendering"], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out_p["loss_metrics"]["loss"], out_b["loss_metrics"]["loss"], rtol=1e-5, atol=1e-7)
    out_p["loss_metrics"]["loss"].backward()
    out_b["loss_metrics"]["loss"].backward()
    grads_b = {n: p.grad for n, p in per_block.named_parameters()}
    for n, p in part.named_parameters():
        m = n
        for old, new in rename.items():
            m = m.replace(f".{old}.", f".{new}.")
        torch.testing.assert_close(p.grad, grads_b[m], rtol=1e-4, atol=1e-7, msg=n)


def test_routing_statistics_definitions():
    from uttt_b200.nvs.blocks import routing_statistics
    reads = torch.tensor([[[6.0, 2.0], [4.0, 4.0]], [[8.0, 0.0], [1.0, 7.0]]])       # [layers, scenes, experts]
    writes = torch.tensor([[[2.0, 2.0], [3.0, 1.0]], [[2.0, 2.0], [0.0, 4.0]]])
    s = routing_statistics(reads, writes, shared_pool=True)
    assert float(s["apply_max_violation_rate"]) == pytest.approx((0.5 + 0.0 + 1.0 + 0.75) / 4)
    assert float(s["apply_min_violation_rate"]) == pytest.approx((0.5 + 0.0 + 1.0 + 0.75) / 4)
    assert float(s["update_max_violation_rate"]) == pytest.approx((0.0 + 0.5 + 0.0 + 1.0) / 4)
    total = reads + writes                                                            # expert shares over the whole pool
    share = total.sum(dim=(0, 1)) / total.sum()
    assert float(s["moe_freq_max"]) == pytest.approx(float(share.max()))
    per_layer = routing_statistics(reads, writes, shared_pool=False)
    flat = total.sum(dim=1).flatten() / total.sum()
    assert float(per_layer["moe_freq_min"]) == pytest.approx(float(flat.min()))
    out = LVSMModel(_cfg())(_batch())
    assert {"apply_min_violation_rate", "update_max_violation_rate", "moe_freq_min"} <= set(out["loss_metrics"])
