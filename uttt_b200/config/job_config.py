"""Job configuration of the language-model trainer: ``--section.key`` flags with a TOML overlay.

Precedence: command line > TOML file (``--job.config_file``) > default, as in the reference
(uttt_llm/flame/config_manager.py:45-66, 927-966).  TOML keys that are not declared flags (for example
``training.expected_global_batch_size`` or an ``[eval]`` table) are kept, so job files can carry extra
settings.  Every section/key of the reference's flag list is declared here.  No flag is silently ignored: each
one is either read by the trainer (``FLAG_READERS`` names where) or, when its value asks for a feature this
framework does not have, rejected by ``_validate`` with the reason (tensor / pipeline / context parallelism,
float8, HSDP replication, parameter resharding, CPU offload of parameters, compiled blocks, torchft).
"""
from __future__ import annotations

import argparse
import sys
from types import SimpleNamespace
from typing import Any, Dict, List, Optional

try:
    import tomllib
except ModuleNotFoundError:  # pragma: no cover
    import tomli as tomllib

_FLAGS: Dict[str, Dict[str, Any]] = {
    "job": dict(config_file=None, dump_folder="./outputs", description="default job", use_for_integration_test=False,
                print_args=False),
    "model": dict(name="uttt", config="", tokenizer_path="", converters=[], print_after_conversion=False),
    "profiling": dict(enable_profiling=False, save_traces_folder="profile_traces", profile_freq=10,
                      enable_memory_snapshot=False, save_memory_snapshot_folder="memory_snapshot"),
    "optimizer": dict(name="AdamW", eps=1e-8, lr=8e-4, beta1=0.9, beta2=0.95, weight_decay=0.1,
                      alpha_weight_decay=True, implementation="fused", early_step_in_backward=False),
    "lr_scheduler": dict(warmup_steps=200, decay_ratio=None, decay_type="linear", lr_min=0.0),
    "training": dict(batch_size=8, seq_len=2048, context_len=2048, varlen=False, gradient_accumulation_steps=1,
                     steps=10000, max_norm=1.0, skip_nan_inf=False, dataset="synthetic", dataset_name=None,
                     dataset_split="train", data_dir=None, data_files=None, data_probs=None, streaming=False,
                     num_workers=4, prefetch_factor=2, data_parallel_replicate_degree=1,
                     data_parallel_shard_degree=-1, enable_cpu_offload=False, tensor_parallel_degree=1,
                     disable_loss_parallel=False, fsdp_reshard_after_forward="default",
                     mixed_precision_param="bfloat16", mixed_precision_reduce="float32", compile=False, gc_freq=50,
                     seed=42, deterministic=False, expected_global_batch_size=None, pin_memory=False,
                     persistent_workers=False, micro_batch_size=None, cuda_graph=False),
    "metrics": dict(log_freq=10, enable_tensorboard=False, disable_color_printing=False, save_tb_folder="tb",
                    save_for_all_ranks=False, enable_wandb=False),
    "experimental": dict(enable_async_tensor_parallel=False, pipeline_parallel_degree=1,
                         pipeline_parallel_split_points=[], pipeline_parallel_schedule="1F1B",
                         pipeline_parallel_schedule_csv="", pipeline_parallel_microbatches=None,
                         enable_compiled_autograd=False, context_parallel_degree=1,
                         context_parallel_rotate_method="allgather", custom_model_path="",
                         expert_parallel_degree=1),
    "checkpoint": dict(enable_checkpoint=False, folder="checkpoint", initial_load_path=None,
                       initial_load_model_weights_only=True, interval=500, model_weights_only=False,
                       save_backend="dcp", last_save_model_weights_only=False, export_dtype="float32",
                       create_seed_checkpoint=False, async_mode="disabled", keep_latest_k=0, load_step=-1,
                       exclude_from_loading=[], interval_type="steps"),
    "activation_checkpoint": dict(mode="selective", selective_ac_option="2", keep_layers=[]),
    "activation_offload": dict(mode="none"),
    "float8": dict(enable_fsdp_float8_all_gather=False, precompute_float8_dynamic_scale_for_fsdp=False,
                   force_recompute_fp8_weight_in_bwd=False, recipe_name=None),
    "comm": dict(init_timeout_seconds=300, train_timeout_seconds=100, trace_buf_size=20000),
    "memory_estimation": dict(enabled=False, disable_fake_mode=False),
    "fault_tolerance": dict(enable=False, replica_id=0, group_size=0, min_replica_size=1),
}


# Where every flag is consumed.  "validate" = its only legal values are checked in JobConfig._validate (the feature
# behind any other value does not exist here); tests assert that this table covers _FLAGS completely.
FLAG_READERS: Dict[str, str] = {
    "job": "lm_trainer.main (dump folder, printing); use_for_integration_test / description: informational",
    "model": "lm_trainer.main (architecture JSON); tokenizer_path: train/data.py; converters: validate",
    "profiling": "lm_trainer.main (torch profiler schedule, memory snapshot)",
    "optimizer": "train/engine.py::EngineConfig (lr, betas, eps, decay); name / implementation / "
                 "early_step_in_backward: validate",
    "lr_scheduler": "train/lr.py::WarmupDecayLR",
    "training": "lm_trainer.main + train/data.py::build_dataloader; data_parallel_replicate_degree: train/engine.py "
                "(hybrid sharding), fsdp_reshard_after_forward: train/engine.py (parameter shards between steps); "
                "other parallel degrees, offload, "
                "compile, mixed precision: validate; gc_freq, deterministic, seed: lm_trainer.main; cuda_graph: "
                "train/engine.py (forward + backward replayed as one CUDA graph)",
    "metrics": "lm_trainer.Metrics",
    "experimental": "validate (degrees); expert_parallel_degree: lm_trainer.main -> memory_expert_parallel",
    "checkpoint": "train/checkpoint.py::CheckpointManager (async_mode included)",
    "activation_checkpoint": "lm_trainer.main (recompute policy of the chunk loop)",
    "activation_offload": "train/engine.py (saved-tensor offload to pinned host memory)",
    "float8": "validate",
    "comm": "train/engine.py::init_distributed (time-outs, flight-recorder size)",
    "memory_estimation": "lm_trainer.main (prints the estimate and stops)",
    "fault_tolerance": "validate",
}


def _str2bool(v: str) -> bool:
    if isinstance(v, bool):
        return v
    if v.lower() in ("1", "true", "yes", "y", "on"):
        return True
    if v.lower() in ("0", "false", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"not a boolean: {v!r}")


def _csv(v: str) -> List[str]:
    return [x for x in v.split(",") if x]


class JobConfig:
    def __init__(self):
        self.parser = argparse.ArgumentParser(description="uttt_b200 language-model trainer")
        for section, flags in _FLAGS.items():
            for key, default in flags.items():
                name = f"--{section}.{key}"
                if isinstance(default, bool):
                    self.parser.add_argument(name, nargs="?", const=True, type=_str2bool, default=None)
                elif isinstance(default, list):
                    self.parser.add_argument(name, type=_csv, default=None)
                elif isinstance(default, (int, float)) and default is not None:
                    self.parser.add_argument(name, type=type(default), default=None)
                else:
                    self.parser.add_argument(name, type=str, default=None)
        # negative spellings kept by the reference
        self.parser.add_argument("--optimizer.no_alpha_weight_decay", action="store_true", default=None)
        self.parser.add_argument("--checkpoint.no_model_weights_only", action="store_true", default=None)
        self.parser.add_argument("--checkpoint.no_initial_load_model_weights_only", action="store_true", default=None)
        self._values: Dict[str, Dict[str, Any]] = {}

    def parse_args(self, args_list: Optional[List[str]] = None) -> "JobConfig":
        args_list = list(sys.argv[1:] if args_list is None else args_list)
        ns = vars(self.parser.parse_args(args_list))
        values = {s: dict(f) for s, f in _FLAGS.items()}
        config_file = ns.get("job.config_file")
        if config_file:
            with open(config_file, "rb") as fh:
                for section, table in tomllib.load(fh).items():
                    if isinstance(table, dict):
                        values.setdefault(section, {}).update(table)     # undeclared keys survive
        for dotted, val in ns.items():
            if val is None:
                continue
            section, key = dotted.split(".", 1)
            if key.startswith("no_"):
                values[section][key[3:]] = False
            else:
                values[section][key] = val
        self._values = values
        for section, table in values.items():
            setattr(self, section, SimpleNamespace(**table))
        self._validate()
        return self

    def _validate(self) -> None:
        t, o, c, e = self.training, self.optimizer, self.checkpoint, self.experimental
        if o.name not in ("AdamW",):
            raise NotImplementedError(f"optimizer.name={o.name!r}: the fused reduce / clip / update kernels implement "
                                      "AdamW (decoupled weight decay) only")
        if o.implementation not in ("fused", "foreach", "for-loop"):
            raise ValueError("optimizer.implementation must be 'fused', 'foreach' or 'for-loop' (all map to the one "
                             "fused kernel here)")
        if o.early_step_in_backward:
            raise NotImplementedError("optimizer.early_step_in_backward: the step needs the global gradient norm "
                                      "for clipping, so it runs after backward")
        world = int(__import__("os").environ.get("WORLD_SIZE", "1"))
        rep = int(t.data_parallel_replicate_degree)
        if rep < 1 or (world > 1 and world % rep != 0):
            raise ValueError(f"training.data_parallel_replicate_degree={rep} does not divide the job size {world}")
        # hybrid sharding: the optimizer state is sharded over world / replicate ranks, replicated `replicate` times
        if t.data_parallel_shard_degree not in (-1, 0) and world > 1 and \
                t.data_parallel_shard_degree * rep != world:
            raise ValueError("training.data_parallel_shard_degree x training.data_parallel_replicate_degree must equal "
                             "the job size (or leave the shard degree at -1)")
        # "always": ranks keep only their parameter shards between steps (gathered once per step: every layer is used
        # by every chunk of the sequence, so re-sharding inside the forward would gather each layer once per chunk)
        if str(t.fsdp_reshard_after_forward) not in ("default", "never", "always"):
            raise ValueError("training.fsdp_reshard_after_forward must be 'default', 'never' or 'always'")
        if t.enable_cpu_offload:
            raise NotImplementedError("training.enable_cpu_offload: parameters and optimizer state live in HBM")
        if t.compile or e.enable_compiled_autograd:
            raise NotImplementedError("training.compile / experimental.enable_compiled_autograd: the hot path is "
                                      "hand-written kernels, there is no traced graph to compile")
        if t.mixed_precision_param != "bfloat16" or t.mixed_precision_reduce != "float32":
            raise NotImplementedError("mixed precision is fixed: bfloat16 parameters / compute, float32 reduction")
        if t.disable_loss_parallel or e.enable_async_tensor_parallel:
            raise NotImplementedError("loss-parallel / async tensor parallel belong to tensor parallelism (degree 1)")
        if self.model.converters:
            raise NotImplementedError(f"model.converters={self.model.converters}: no module converters (float8) here")
        if c.async_mode not in ("disabled", "async", "async_with_pinned_mem"):
            raise ValueError("checkpoint.async_mode must be 'disabled', 'async' or 'async_with_pinned_mem'")
        if c.interval_type != "steps":
            raise NotImplementedError("checkpoint.interval_type must be 'steps'")
        if self.activation_checkpoint.mode not in ("none", "selective", "full"):
            raise ValueError("activation_checkpoint.mode must be 'none', 'selective' or 'full'")
        if self.activation_offload.mode not in ("none", "offload"):
            raise ValueError("activation_offload.mode must be 'none' or 'offload'")
        if self.fault_tolerance.enable:
            raise NotImplementedError("fault_tolerance.enable: torchft is not available; failures are handled by "
                                      "step skipping, bounded waits and atomic checkpoints")
        if self.float8.precompute_float8_dynamic_scale_for_fsdp or self.float8.force_recompute_fp8_weight_in_bwd \
                or self.float8.recipe_name:
            raise NotImplementedError("float8 training is not implemented")
        if self.training.tensor_parallel_degree != 1:
            raise NotImplementedError("tensor_parallel_degree > 1: the uTTT model families have no tensor-parallel plan")
        if self.experimental.pipeline_parallel_degree != 1:
            raise NotImplementedError("pipeline parallelism is not implemented for the recurrent chunk schedule")
        if self.experimental.context_parallel_degree != 1:
            raise NotImplementedError("context parallelism is not needed: state is constant-size, attention is windowed")
        if self.float8.enable_fsdp_float8_all_gather:
            raise NotImplementedError("float8 all-gather is not implemented")
        if self.checkpoint.save_backend not in ("dcp", "rank0_model_only"):
            raise ValueError("checkpoint.save_backend must be 'dcp' or 'rank0_model_only'")

    def to_dict(self) -> Dict[str, Dict[str, Any]]:
        return {s: dict(t) for s, t in self._values.items()}
