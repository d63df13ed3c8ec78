"""Job configuration of the language-model trainer: ``--section.key`` flags with a TOML overlay.

Precedence: command line > TOML file (``--job.config_file``) > default, as in the reference
(uttt_llm/flame/config_manager.py:45-66, 927-966).  TOML keys that are not declared flags (for example
``training.expected_global_batch_size`` or an ``[eval]`` table) are kept, so job files can carry extra
settings.  Every section/key of the reference's flag list is declared here; options whose feature this
framework does not implement (tensor / pipeline / context parallel degrees above 1, float8) are accepted
and rejected with a clear error at trainer start.
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
                     persistent_workers=False, micro_batch_size=None),
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
    "activation_checkpoint": dict(mode="selective", selective_ac_option="2"),
    "activation_offload": dict(mode="none"),
    "float8": dict(enable_fsdp_float8_all_gather=False, precompute_float8_dynamic_scale_for_fsdp=False,
                   force_recompute_fp8_weight_in_bwd=False, recipe_name=None),
    "comm": dict(init_timeout_seconds=300, train_timeout_seconds=100, trace_buf_size=20000),
    "memory_estimation": dict(enabled=False, disable_fake_mode=False),
    "fault_tolerance": dict(enable=False, replica_id=0, group_size=0, min_replica_size=1),
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
        assert self.model.config or self.job.use_for_integration_test or True
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
