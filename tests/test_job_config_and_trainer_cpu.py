import json
import os

import pytest
import torch

from uttt_b200.config import named_config
from uttt_b200.config.job_config import JobConfig
from uttt_b200.train import lm_trainer
from uttt_b200.train.lr import WarmupDecayLR


def _write(tmp_path, toml_extra=""):
    model = tmp_path / "model.json"
    model.write_text(named_config("tiny-uttt-moe").to_json_string())
    job = tmp_path / "job.toml"
    job.write_text(f"""
[job]
dump_folder = "{tmp_path}/out"
[training]
batch_size = 2
seq_len = 128
steps = 3
expected_global_batch_size = 2
dataset = "synthetic"
skip_nan_inf = true
{toml_extra}
[optimizer]
lr = 1e-3
[lr_scheduler]
warmup_steps = 1
decay_type = "cosine"
lr_min = 0.1
[checkpoint]
enable_checkpoint = true
interval = 2
keep_latest_k = 2
[metrics]
log_freq = 1
[eval]
anything = "kept"
""")
    return str(job), str(model)


def test_precedence_cmdline_over_toml_over_default(tmp_path):
    job, model = _write(tmp_path)
    cfg = JobConfig().parse_args(["--job.config_file", job, "--model.config", model, "--training.steps", "7",
                                  "--checkpoint.no_model_weights_only"])
    assert cfg.training.steps == 7                       # command line wins
    assert cfg.training.seq_len == 128                   # TOML over default
    assert cfg.optimizer.beta2 == 0.95                   # default
    assert cfg.training.expected_global_batch_size == 2  # undeclared-in-reference key survives
    assert cfg.to_dict()["eval"]["anything"] == "kept"
    assert cfg.checkpoint.model_weights_only is False


def test_unsupported_parallelism_is_rejected(tmp_path):
    job, model = _write(tmp_path)
    with pytest.raises(NotImplementedError):
        JobConfig().parse_args(["--job.config_file", job, "--training.tensor_parallel_degree", "2"])
    with pytest.raises(NotImplementedError):
        JobConfig().parse_args(["--job.config_file", job, "--experimental.pipeline_parallel_degree", "2"])


def test_global_batch_guard(tmp_path):
    job, model = _write(tmp_path)
    cfg = JobConfig().parse_args(["--job.config_file", job, "--model.config", model, "--training.batch_size", "3"])
    with pytest.raises(ValueError):
        lm_trainer.check_global_batch(cfg, 1)


def test_train_checkpoint_and_resume(tmp_path):
    job, model = _write(tmp_path)
    args = ["--job.config_file", job, "--model.config", model]
    state = lm_trainer.main(JobConfig().parse_args(args))
    assert state.step == 3 and len(state.global_avg_losses) == 3
    ckpt_dir = tmp_path / "out" / "checkpoint"
    assert sorted(os.listdir(ckpt_dir)) == ["step-2", "step-3"]
    lines = [json.loads(l) for l in open(tmp_path / "out" / "metrics.jsonl")]
    assert lines[-1]["step"] == 3 and lines[-1]["loss"] < lines[0]["loss"] + 0.5
    state2 = lm_trainer.main(JobConfig().parse_args(args + ["--training.steps", "4"]))
    assert state2.step == 4 and state2.log_steps[:3] == [1, 2, 3]     # resumed from step 3, history restored


def test_lr_schedule_shapes():
    s = WarmupDecayLR(1.0, 100, warmup_steps=10, decay_type="cosine", lr_min=0.1)
    assert s.factor(0) < s.factor(5) < s.factor(9) <= 1.0
    assert abs(s.factor(10) - 1.0) < 1e-6 and abs(s.factor(100) - 0.1) < 1e-6
    lin = WarmupDecayLR(1.0, 100, warmup_steps=0, decay_type="linear", lr_min=0.0, decay_ratio=0.2)
    assert lin.factor(50) == 1.0 and lin.factor(90) == pytest.approx(0.5)
