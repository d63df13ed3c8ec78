"""Writes the configuration tree under ``configs/``:  ``python -m uttt_b200.tools.make_configs``.

* ``configs/lm/main/{124M,760M}/<model>.json`` - architecture files of every language-model family at the two paper
  scales (the shapes shipped with the reference, uttt_llm/configs/main), plus ``configs/lm/named/*.json`` for the
  benchmark-named shapes and ``configs/lm/balancing/*`` for the loss-free-rate / scope / router-alpha sweeps;
* ``configs/lm/exp/train_{124M,760M}_32k.toml`` and ``eval_ptl.toml`` - job files (global batch 32 at 32K);
* ``configs/nvs/<study>/<data>/<name>.yaml`` - view-synthesis runs (ownership ladder, capacity, width, topology,
  dense widths, schedule, transformer and delta-rule references, 242M scale ladder).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict

import yaml

from ..config.lm_config import _COMMON_UTTT, config_from_dict, named_config

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "configs")

SCALES = {"124M": dict(hidden_size=768, num_hidden_layers=12, num_heads=12),
          "760M": dict(hidden_size=1536, num_hidden_layers=24, num_heads=24)}
MOE = dict(memory_router_share_mode="per_layer", memory_update_aggregate_write=True,
           memory_aggregate_momentum_mode="pool_mean", memory_update_backward_mode="full",
           memory_lb_mode="loss_free", memory_lb_scope="pool", fw_num_heads=4, fw_inter_multi=1, w0_w2_low_rank=32)


def lm_shapes(scale: str) -> Dict[str, Dict[str, Any]]:
    base = dict(_COMMON_UTTT, **SCALES[scale], window_size=4096, chunk_size=4096)
    small = scale == "124M"
    out = {
        "uttt_moe": dict(base, **MOE, model_type="uttt_moe", memory_num_experts=48 if small else 96,
                         memory_num_active_experts=1, memory_loss_free_update_rate=3e-5 if small else 1e-3),
        "ttt_moe_lb": {**base, **MOE, **dict(model_type="ttt_moe_lb", memory_pool_mode="per_layer",
                                             memory_update_aggregate_write=False,
                                             memory_aggregate_momentum_mode="none", memory_num_experts=4,
                                             memory_lb_scope="layer", memory_loss_free_update_rate=1e-5)},
        "ttt_moe_no_lb": {**base, **MOE, **dict(model_type="ttt_moe_no_lb", memory_pool_mode="per_layer",
                                                memory_update_aggregate_write=False,
                                                memory_aggregate_momentum_mode="none", memory_num_experts=4,
                                                memory_lb_scope="layer", memory_lb_mode="loss",
                                                memory_lb_loss_alpha=0.0)},
        # w0 / w2 of the per-layer dense families start as identity + a rank-32 product
        "ttt_dense": dict(base, model_type="ttt_dense", fw_num_heads=4, fw_inter_multi=1, w0_w2_low_rank=32),
        "lact": dict(base, model_type="lact_swiglu", num_lact_heads=4, inter_multi=1, lact_chunk_size=4096,
                     w0_w2_low_rank=32, num_attn_heads=SCALES[scale]["num_heads"]),
        "transformer": dict(base, model_type="transformer", use_memory_block=False, window_size=None),
        "transformer_swa": dict(base, model_type="transformer", use_memory_block=False),
    }
    # the bounded-state baselines, sized to the parameter budget of the fast-weight models: no short convolutions,
    # the MLP narrowed where the mixer itself carries more parameters (gate, decay, state projections)
    h = SCALES[scale]["hidden_size"]
    mixers = {
        "deltanet": dict(use_short_conv=False),
        "gated_deltanet": dict(use_short_conv=False, use_gate=True, hidden_ratio=3.5),
        "kda": dict(use_short_conv=False, hidden_ratio=None, intermediate_size={768: 1984, 1536: 4032}[h]),
        "mamba2": dict(hidden_ratio=3.5, intermediate_size=h * 3 // 2, state_size=h * 3 // 4, chunk_size=256),
        "mom": dict(use_short_conv=False, use_gate=True, hidden_ratio=3.5, num_memories=4, topk_memories=1),
    }
    for mixer, extra in mixers.items():
        out[f"{mixer}_swa"] = dict(base, model_type=f"{mixer}_swa", use_memory_block=False, mixer_head_dim=64, **extra)
    if small:
        for r in (1, 2, 4, 6):
            out[f"uttt_dense_r{r}"] = dict(base, model_type="uttt_dense", fw_num_heads=4, uttt_dense_r=r,
                                           w0_w2_low_rank=0)
    return out


def job_toml(scale: str) -> str:
    bs = {"124M": 4, "760M": 2}[scale]
    steps = {"124M": 10240, "760M": 40960}[scale]
    return f"""# {scale} @ 32K context: per-device batch {bs}; the global batch must be 32 sequences.
[job]
dump_folder = "runs"
print_args = true

[training]
batch_size = {bs}
seq_len = 32768
context_len = 32768
gradient_accumulation_steps = 1
expected_global_batch_size = 32
steps = {steps}
max_norm = 1.0
skip_nan_inf = true
data_parallel_shard_degree = -1
tensor_parallel_degree = 1
dataset = "synthetic"
seed = 42
fsdp_reshard_after_forward = "never"

[optimizer]
name = "AdamW"
eps = 1e-15
lr = 1e-3

[lr_scheduler]
warmup_steps = 1024
decay_type = "cosine"
lr_min = 0.1

[checkpoint]
enable_checkpoint = true
folder = "checkpoint"
interval = 2048
keep_latest_k = 2
load_step = -1
export_dtype = "float32"

[profiling]
enable_profiling = false
profile_freq = 512

[metrics]
log_freq = 10

[experimental]
context_parallel_degree = 1
pipeline_parallel_degree = 1
"""


def nvs_yaml(name: str, block_type: str, params: Dict[str, Any], dim=512, layers=8, size=256, batch=32,
             views=12, total=128, **training) -> Dict[str, Any]:
    tr = dict(total_batch_size=total, grad_accum_steps=1, grad_clip_norm=1.0, may_skip_gradnorm_after=1000,
              allowed_gradnorm_factor=5, dataset="synthetic", num_views=views, eval_num_views=24,
              batch_size_per_gpu=batch, num_workers=16, lpips_loss_weight=0.0, max_fwdbwd_passes=20000, lr=4e-4,
              beta1=0.9, beta2=0.95, weight_decay=0.05, warmup=2500, vis_every=1000, print_every=20,
              checkpoint_every=500, wandb_log_every=50, wandb_offline=False, prefetch_factor=4)
    tr.update(training)
    return {"exp_name": name, "model": {"class_name": "uttt_b200.nvs.model.LVSMModel", "image_size": size,
                                        "patch_size": 8, "dim": dim, "layers": layers,
                                        "block_config": {"type": block_type, "params": params}}, "training": tr}


def nvs_configs() -> Dict[str, Dict[str, Any]]:
    moe = "uttt_nvs.models.uttt_moe_block.MemoryModel"
    dense = "uttt_nvs.models.uttt_dense_block.MemoryModel"
    base = dict(attn_head_dim=64, fw_head_dim=64, inter_multi=3, fw_inter_multi=1, use_muon=False, num_experts=64,
                num_active_experts=1, router_alpha=1.0, load_balancing_loss_alpha=1e-5, l2_norm=True,
                pool_mode="shared", router_share_mode="share_all", aggregate_write=True)
    out = {}
    for data in ("obj", "dl3dv"):
        out[f"ownership/{data}/uttt_moe_e64a1"] = nvs_yaml(f"uttt_moe_e64a1_{data}", moe, dict(base))
        out[f"ownership/{data}/ttt_moe_e8a1"] = nvs_yaml(
            f"ttt_moe_e8a1_{data}", moe, dict(base, num_experts=8, pool_mode="per_block", aggregate_write=False,
                                              router_share_mode="per_layer"))
        out[f"ownership/{data}/ttt_moe_e4a1"] = nvs_yaml(
            f"ttt_moe_e4a1_{data}", moe, dict(base, num_experts=4, pool_mode="per_block", aggregate_write=False,
                                              router_share_mode="per_layer"))
        out[f"ownership/{data}/uttt_dense_r1"] = nvs_yaml(f"uttt_dense_r1_{data}", dense, dict(
            attn_head_dim=64, fw_head_dim=64, inter_multi=3, fw_inter_multi=1, use_muon=False, l2_norm=True,
            aggregate_write=True))
        # TTT-Dense: every block owns its head-wise fast weights (no sharing, no aggregate)
        out[f"ownership/{data}/ttt_dense"] = nvs_yaml(f"ttt_dense_{data}", "uttt_nvs.models.ttt_dense_block.MemoryModel", dict(
            attn_head_dim=64, fw_head_dim=64, inter_multi=3, fw_inter_multi=1, l2_norm=True, use_muon=False))
        for e in (8, 16, 32, 64, 128, 256):
            out[f"capacity/{data}/uttt_moe_e{e}a1"] = nvs_yaml(f"uttt_moe_e{e}a1_{data}", moe, dict(base, num_experts=e))
        for k in (2, 4):
            out[f"topology/{data}/uttt_moe_e64a{k}"] = nvs_yaml(f"uttt_moe_e64a{k}_{data}", moe,
                                                               dict(base, num_active_experts=k))
        out[f"topology/{data}/uttt_moe_e64a1_perlayer_router"] = nvs_yaml(
            f"uttt_moe_e64a1_plr_{data}", moe, dict(base, router_share_mode="per_layer"))
        out[f"topology/{data}/uttt_moe_e64a1_chained"] = nvs_yaml(
            f"uttt_moe_e64a1_chained_{data}", moe, dict(base, aggregate_write=False))
        out[f"topology/{data}/uttt_moe_e64a1_p2"] = nvs_yaml(
            f"uttt_moe_e64a1_p2_{data}", "uttt_nvs.models.uttt_moe_partitioned.MemoryModel", dict(base, num_partitions=2))
        for m in (2, 4):
            out[f"width/{data}/uttt_moe_e64a1_w{m}"] = nvs_yaml(f"uttt_moe_e64a1_w{m}_{data}", moe,
                                                               dict(base, fw_inter_multi=m))
        for r in (2, 4, 8):
            out[f"dense/{data}/uttt_dense_r{r}"] = nvs_yaml(f"uttt_dense_r{r}_{data}", dense, dict(
                attn_head_dim=64, fw_head_dim=64, inter_multi=3, fw_inter_multi=r, use_muon=False, l2_norm=True,
                aggregate_write=True))
        # the released studies, under the names of the reference's files
        dense_base = dict(attn_head_dim=64, fw_head_dim=64, inter_multi=3, fw_inter_multi=1, use_muon=False, l2_norm=True,
                          aggregate_write=True)
        for e in (32, 64):
            for k in (1, 2, 4, 8):
                out[f"width/{data}/uttt_moe_e{e}a{k}"] = nvs_yaml(f"uttt_moe_e{e}a{k}_{data}", moe,
                                                                 dict(base, num_experts=e, num_active_experts=k))
            out[f"topology/{data}/uttt_moe_e{e}a1"] = nvs_yaml(f"uttt_moe_e{e}a1_{data}", moe, dict(base, num_experts=e))
            for pools in (2, 4):
                out[f"topology/{data}/uttt_moe_p{pools}_e{e}"] = nvs_yaml(
                    f"uttt_moe_p{pools}_e{e}_{data}", "uttt_nvs.models.uttt_moe_partitioned.MemoryModel",
                    dict(base, num_experts=e, num_shared_pools=pools))
        for width, pools in ((1, 2), (1, 4), (2, 4), (4, 2)):
            out[f"topology/{data}/uttt_dense_w{width}_p{pools}"] = nvs_yaml(
                f"uttt_dense_w{width}_p{pools}_{data}", "uttt_nvs.models.uttt_dense_partitioned.MemoryModel",
                dict(dense_base, fw_inter_multi=width, num_shared_pools=pools, pool_mode="shared"))
        out[f"dense/{data}/uttt_dense_r1"] = nvs_yaml(f"uttt_dense_r1_{data}", dense, dict(dense_base))
        out[f"schedule/{data}/uttt_moe_e64a1"] = nvs_yaml(f"uttt_moe_e64a1_{data}", moe, dict(base))
        out[f"schedule/{data}/uttt_moe_e64a1_chained"] = nvs_yaml(f"uttt_moe_e64a1_chained_{data}", moe,
                                                                 dict(base, aggregate_write=False))
        out[f"schedule/{data}/uttt_moe_4in2out"] = nvs_yaml(f"uttt_moe_4in2out_{data}", moe, dict(base), views=6)
        out[f"schedule/{data}/uttt_moe_4in2out"]["model"].update(view_layout="inputs_then_targets", num_input_views=4)
        out[f"transformer/{data}/transformer"] = nvs_yaml(
            f"transformer_{data}", "uttt_nvs.models.transformer_block.MemoryModel",
            dict(attn_head_dim=64, inter_multi=3, transformer_version="v0", vi_rms_norm=True,
                 pre_vi_source="xi_memory_in", use_separate_last_to_kv=False), num_workers=8)
        # widths of the slow MLP chosen so that the baselines match the parameter count of the fast-weight models
        out[f"reference/{data}/deltanet"] = nvs_yaml(
            f"deltanet_{data}", "uttt_nvs.models.deltanet_block.MemoryModel",
            dict(attn_head_dim=64, inter_multi=3.09375, fw_num_heads=8, expand_k=1.0, expand_v=1.0, use_beta=True,
                 use_short_conv=False, conv_size=4, conv_bias=False, qk_activation="silu", qk_norm="l2",
                 use_output_gate=False, allow_neg_eigval=False, noise_repeat=1, repeat_function="repeat",
                 use_muon=False), batch=16, num_workers=8)
        out[f"reference/{data}/gated_deltanet"] = nvs_yaml(
            f"gated_deltanet_{data}", "uttt_nvs.models.gated_deltanet_block.MemoryModel",
            dict(attn_head_dim=64, inter_multi=2.75, fw_num_heads=8, expand_v=1.0, use_short_conv=False, conv_size=4,
                 conv_bias=False, use_output_gate=True, noise_repeat=1, repeat_function="repeat", use_muon=False),
            batch=16, num_workers=8)
    big = dict(base, num_experts=96, fw_head_dim=192, fw_inter_multi=2, attn_head_dim=64, apply_ckpt_group=6,
               offload_master_states=True)
    # resolution curriculum of the large model: 256 from scratch, then 512 and 1024 from the previous stage's weights
    # with a fresh optimizer at a small constant-peak rate; perceptual loss after an l2-only warm-up
    stages = {256: dict(batch=8, total=512, max_fwdbwd_passes=81038),
              512: dict(batch=2, total=128, max_fwdbwd_passes=70000, lr=1e-5, reset_training_state=True,
                        load_optimizer_state_when_reset_training_state=False),
              1024: dict(batch=1, total=64, max_fwdbwd_passes=4500, lr=1e-5, reset_training_state=True,
                         load_optimizer_state_when_reset_training_state=False)}
    for size, stage in stages.items():
        out[f"scale/obj/uttt_moe_large_{size}"] = nvs_yaml(
            f"uttt_moe_large_{size}_obj", moe, dict(big), dim=768, layers=24, size=size, num_workers=4,
            perceptual_loss_weight=0.5, l2_warmup_steps=4000, round_max_fwdbwd_passes_to_epoch=False, **stage)
    out["named/uttt_moe_256_4in2out"] = nvs_yaml(
        "uttt_moe_256_4in2out", moe, dict(base, num_experts=16, num_active_experts=2, fw_head_dim=64), dim=768,
        layers=24, size=256, batch=16, total=128, views=6)
    out["named/uttt_moe_256_4in2out"]["model"].update(view_layout="inputs_then_targets", num_input_views=4)
    return out


def eval_registries() -> Dict[str, Dict[str, Any]]:
    """``experiments.yaml`` (the evaluated fast-weight models and linear baselines on both test sets) and
    ``experiments_transformer.yaml`` (the transformer, whose attention gap must be declared null)."""
    defaults = {"checkpoint_root": "/PATH/TO/CHECKPOINTS", "output_root": "/PATH/TO/EVAL_OUTPUTS",
                "wandb": {"entity": "YOUR_WANDB_ENTITY", "project": "YOUR_WANDB_PROJECT"}, "seed": 9595, "num_views": 24}
    datasets = [
        {"id": "gso", "display_name": "Objaverse/GSO",
         "local_manifest": "/PATH/TO/MANIFESTS/gso_v0.1_instant3d_test_localssd.txt",
         "view_manifest": "/PATH/TO/MANIFESTS/gso_views_seed9595_v24.json", "expected_scenes": 1019,
         "expected_rows": 1019 * 23},
        {"id": "dl3dv", "display_name": "DL3DV", "local_manifest": "/PATH/TO/MANIFESTS/dl3dv10k_benchmark_local.txt",
         "view_manifest": "/PATH/TO/MANIFESTS/dl3dv_views_seed9595_v24.json", "expected_scenes": 140,
         "expected_rows": 140 * 23}]
    domain = {"gso": ("obj", "object", 24476), "dl3dv": ("dl3dv", "dl3dv", 20046)}

    def entry(ds, study, model, paper, impl, group, label, **extra):
        folder, ckpt_folder, step = domain[ds]
        return {"id": f"{ds}_{model}", "dataset": ds, "model": model, "paper_model": paper,
                "config": f"configs/nvs/{study}/{folder}/{model}.yaml", "checkpoint": f"{ckpt_folder}/{model}/checkpoint.pt",
                "checkpoint_step": step, "checkpoint_impl": impl, "group": group, "display_name": label, **extra}

    def core(ds):
        # the per-block routed model was trained with another implementation on DL3DV: the label tells them apart
        rows = [entry(ds, "ownership", "ttt_dense", "TTT-Dense", "ttt_dense", "ttt_dense", "TTT-Dense")]
        rows += [entry(ds, "ownership", f"ttt_moe_e{e}a1", "TTT-MoE", "ttt_moe" if ds == "gso" else "ttt_moe_alt",
                       "ttt_moe", f"TTT-MoE-e{e}a1") for e in (4, 8)]
        rows += [entry(ds, "dense", f"uttt_dense_r{r}", "uTTT-Dense", "uttt_dense", "uttt_dense", f"uTTT-Dense-r{r}")
                 for r in (1, 2, 4, 8)]
        rows += [entry(ds, "capacity", f"uttt_moe_e{e}a1", "uTTT-MoE", "uttt_moe", "uttt_moe", f"uTTT-MoE-e{e}a1")
                 for e in (8, 16, 32, 64)]
        rows += [entry(ds, "width", f"uttt_moe_e{e}a{k}", "uTTT-MoE", "uttt_moe", "uttt_moe", f"uTTT-MoE-e{e}a{k}")
                 for e in (32, 64) for k in (2, 4, 8)]
        return rows

    def studies(ds):
        rows = [entry(ds, "topology", f"uttt_moe_p{p}_e{e}", "uTTT-MoE", "uttt_moe_partitioned", "uttt_moe",
                      f"uTTT-MoE-e{e // p}-p{p}") for e in (32, 64) for p in (2, 4)]
        rows += [entry(ds, "topology", f"uttt_dense_w{w}_p{p}", "uTTT-Dense", "uttt_dense_partitioned", "uttt_dense",
                       f"uTTT-Dense-w{w}-p{p}") for w, p in ((4, 2), (2, 4), (1, 2), (1, 4))]
        rows.append(entry(ds, "schedule", "uttt_moe_e64a1_chained", "uTTT-MoE", "uttt_moe", "uttt_moe",
                          "uTTT-MoE-e64a1 (chained write)"))
        rows.append(entry(ds, "reference", "deltanet", "DeltaNet", "deltanet", "reference", "DeltaNet"))
        rows.append(entry(ds, "reference", "gated_deltanet", "Gated DeltaNet", "gated_deltanet", "reference",
                          "Gated DeltaNet"))
        return rows

    main = core("gso") + core("dl3dv") + studies("gso") + studies("dl3dv")
    transformer = []
    for ds, ckpt, step in (("dl3dv", "dl3dv_vgapnull", 20000), ("gso", "objaverse_vgapnull", 24000)):
        row = entry(ds, "transformer", "transformer", "Transformer", "transformer", "transformer", "Transformer",
                    expected_v_gap=None, evaluation_class="formal_vgap_null")
        row.update(id=f"{ds}_transformer_vgapnull", checkpoint=f"{ckpt}/checkpoint.pt", checkpoint_step=step)
        transformer.append(row)
    return {"experiments.yaml": {"version": 1, "defaults": defaults, "datasets": datasets, "experiments": main},
            "experiments_transformer.yaml": {"version": 1, "defaults": defaults, "datasets": datasets,
                                             "experiments": transformer}}


def main() -> None:
    for scale in SCALES:
        for name, cfg in lm_shapes(scale).items():
            path = os.path.join(ROOT, "lm", "main", scale, f"{name}.json")
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as fh:
                fh.write(config_from_dict(cfg).to_json_string())
        path = os.path.join(ROOT, "lm", "exp", f"train_{scale}_32k.toml")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as fh:
            fh.write(job_toml(scale))
    with open(os.path.join(ROOT, "lm", "exp", "eval_ptl.toml"), "w") as fh:
        fh.write('[job]\ndump_folder = "runs/eval"\n\n[training]\nbatch_size = 1\nseq_len = 32768\ndataset = "synthetic"\n\n'
                 '[eval]\nptl_start = 30000\nmax_batches = 64\n')
    # the LaCT baseline's own published shapes (24 layers; window and chunk 2048; w0 / w2 low rank 32), with and
    # without Newton-Schulz, and the fp32-state variant of the 760M model
    lact = dict(lm_shapes("760M")["lact"], window_size=2048, chunk_size=2048, lact_chunk_size=2048)
    for name, extra in {
        "760M_lact_swiglu_nh4_fwlow_rank_momentum": dict(use_muon=False),
        "760M_lact_swiglu_nh4_fwlow_rank_momentum_muon": dict(use_muon=True),
        "760M_lact_swiglu_nh4_fwlow_rank_momentum_fused_kernel": dict(use_muon=False, use_fused_kernel=True,
                                                                      fp32_states=True, no_v_silu=True),
        "3B_lact_swiglu_nh4_fwlow_rank_momentum": dict(use_muon=False, hidden_size=3072, num_heads=24, num_attn_heads=24),
        "3B_lact_swiglu_nh4_fwlow_rank_momentum_muon": dict(use_muon=True, hidden_size=3072, num_heads=24,
                                                            num_attn_heads=24),
    }.items():
        path = os.path.join(ROOT, "lm", "lact", f"{name}.json")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as fh:
            fh.write(config_from_dict(dict(lact, **extra)).to_json_string())
    os.makedirs(os.path.join(ROOT, "lm", "named"), exist_ok=True)
    for name in ("760M-uttt-moe", "124M-uttt-moe", "124M-uttt-dense", "tiny-uttt-moe"):
        with open(os.path.join(ROOT, "lm", "named", f"{name}.json"), "w") as fh:
            fh.write(named_config(name).to_json_string())
    for scale in SCALES:
        base = lm_shapes(scale)["uttt_moe"]
        sweeps = {f"rate_{r:g}": dict(memory_loss_free_update_rate=r) for r in (1e-5, 1e-4, 1e-3, 1e-2)}
        sweeps.update({"scope_layer": dict(memory_lb_scope="layer"), "aux_loss": dict(memory_lb_mode="loss", memory_lb_loss_alpha=0.01),
                       "no_balancing": dict(memory_lb_mode="none"), "alpha_0.5": dict(memory_router_alpha=0.5),
                       "alpha_2": dict(memory_router_alpha=2.0)})
        for name, over in sweeps.items():
            path = os.path.join(ROOT, "lm", "balancing", scale, f"uttt_moe_{name}.json")
            os.makedirs(os.path.dirname(path), exist_ok=True)
            with open(path, "w") as fh:
                fh.write(config_from_dict(dict(base, **over)).to_json_string())
    # the released balancing studies, under the names of the reference's files: loss-free update rates for the
    # layer-local family (expert count / active experts), auxiliary-loss weights for the family without loss-free
    # balancing, and rate / scope / router-temperature sweeps of the universal pool
    def rate_tag(r: float) -> str:
        m, e = f"{r:.0e}".split("e")
        return f"{m}e{int(e)}"
    for scale in SCALES:
        shapes = lm_shapes(scale)
        small = scale == "124M"
        named = {}
        lb_grid = ({(4, 1): (1e-4, 3e-5, 3e-6), (4, 2): (1e-4, 1e-5, 3e-5, 3e-6), (8, 1): (1e-4, 1e-5, 3e-5, 3e-6)}
                   if small else {(4, 1): (1e-4, 3e-5)})
        for (e, k), rates in lb_grid.items():
            for r in rates:
                named[f"ttt_moe_lb_e{e}a{k}_lossfree_u{rate_tag(r)}"] = dict(
                    shapes["ttt_moe_lb"], memory_num_experts=e, memory_num_active_experts=k,
                    memory_loss_free_update_rate=r)
        for a in ((1e-5, 1e-6) if small else (1e-4, 1e-5, 3e-5)):
            named[f"ttt_moe_no_lb_e4a1_lb{rate_tag(a)}"] = dict(shapes["ttt_moe_no_lb"], memory_lb_loss_alpha=a)
        named["ttt_moe_no_lb_e4a2_lb0"] = dict(shapes["ttt_moe_no_lb"], memory_num_active_experts=2)
        named["ttt_moe_no_lb_e8a1_lb0"] = dict(shapes["ttt_moe_no_lb"], memory_num_experts=8)
        e = shapes["uttt_moe"]["memory_num_experts"]
        tail = "agg_poolmean_lr1_full_router_per_layer"
        if small:
            grid = [("layer", r, None) for r in (1e-3, 1e-4, 1e-5, 3e-4, 3e-5)] + \
                   [("pool", r, None) for r in (1e-3, 1e-4, 1e-5, 3e-4)]
        else:
            grid = [("pool", r, None) for r in (1e-4, 1e-5, 3e-4, 3e-5)] + \
                   [("pool", 1e-4, 2), ("pool", 1e-4, 4), ("pool", 3e-4, 2), ("pool", 3e-5, 2)]
        for scope, r, alpha in grid:
            name = f"uttt_moe_e{e}a1_lossfree_{scope}_u{rate_tag(r)}" + (f"_alpha{alpha}" if alpha else "") + f"_{tail}"
            over = dict(memory_lb_scope=scope, memory_loss_free_update_rate=r)
            if alpha:
                over["memory_router_alpha"] = float(alpha)
            named[name] = dict(shapes["uttt_moe"], **over)
        for name, cfg in named.items():
            with open(os.path.join(ROOT, "lm", "balancing", scale, f"{name}.json"), "w") as fh:
                fh.write(config_from_dict(cfg).to_json_string())
    for rel, cfg in nvs_configs().items():
        path = os.path.join(ROOT, "nvs", rel + ".yaml")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as fh:
            yaml.safe_dump(cfg, fh, sort_keys=False)
    # evaluation registries, in the reference's layout and with its experiment ids, checkpoint paths and labels
    for fname, doc in eval_registries().items():
        os.makedirs(os.path.join(ROOT, "nvs", "eval"), exist_ok=True)
        with open(os.path.join(ROOT, "nvs", "eval", fname), "w") as fh:
            # one table row per dataset / experiment: easier to scan and to diff than a block per entry
            fh.write("# Evaluation registry (layout: uttt_b200/nvs/eval/registry.py).  Generated by "
                     "uttt_b200/tools/make_configs.py.\n")
            head = {k: v for k, v in doc.items() if k not in ("datasets", "experiments")}
            fh.write(yaml.safe_dump(head, sort_keys=False))
            for key in ("datasets", "experiments"):
                fh.write(f"{key}:\n")
                for row in doc[key]:
                    line = yaml.safe_dump(row, default_flow_style=True, sort_keys=False, width=10 ** 6).strip()
                    fh.write(f"  - {line}\n")
    print(f"wrote configs under {ROOT}")


if __name__ == "__main__":
    main()
