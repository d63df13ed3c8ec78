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


def test_every_flag_has_a_reader_or_is_rejected(tmp_path):
    from uttt_b200.config.job_config import FLAG_READERS, _FLAGS
    assert set(FLAG_READERS) == set(_FLAGS)
    job, model = _write(tmp_path)
    base = ["--job.config_file", job, "--model.config", model]
    for bad in (["--training.compile"], ["--optimizer.name", "Lion"], ["--optimizer.early_step_in_backward"],
                ["--training.enable_cpu_offload"],
                ["--fault_tolerance.enable"],
                ["--training.mixed_precision_param", "float16"], ["--model.converters", "float8"],
                ["--experimental.enable_compiled_autograd"]):
        with pytest.raises(NotImplementedError):
            JobConfig().parse_args(base + bad)
    for bad in (["--checkpoint.async_mode", "sometimes"], ["--activation_checkpoint.mode", "maybe"],
                ["--activation_offload.mode", "disk"], ["--training.data_parallel_replicate_degree", "0"],
                ["--training.fsdp_reshard_after_forward", "sometimes"]):
        with pytest.raises(ValueError):
            JobConfig().parse_args(base + bad)
    # hybrid sharding is accepted when it divides the job size (a single process accepts any positive degree here;
    # the engine checks it against the real job)
    JobConfig().parse_args(base + ["--training.data_parallel_replicate_degree", "2"])
    # the reference's own job file values are all accepted
    JobConfig().parse_args(base + ["--training.fsdp_reshard_after_forward", "never", "--activation_checkpoint.mode",
                                   "none", "--activation_checkpoint.selective_ac_option", "1"])


def test_async_checkpoint_gc_and_param_check(tmp_path, capsys):
    job, model = _write(tmp_path)
    args = ["--job.config_file", job, "--model.config", model, "--checkpoint.async_mode", "async",
            "--training.gc_freq", "1", "--job.print_args", "--training.deterministic"]
    state = lm_trainer.main(JobConfig().parse_args(args))
    assert state.step == 3
    assert sorted(os.listdir(tmp_path / "out" / "checkpoint")) == ["step-2", "step-3"]   # the writer was joined
    out = capsys.readouterr().out
    assert "[param-check] model.embeddings.weight" in out and "std=" in out
    torch.use_deterministic_algorithms(False)


def test_memory_estimate_stops_before_training(tmp_path, capsys):
    job, model = _write(tmp_path)
    state = lm_trainer.main(JobConfig().parse_args(["--job.config_file", job, "--model.config", model,
                                                    "--memory_estimation.enabled"]))
    assert state.step == 0 and "[memory-estimate]" in capsys.readouterr().out
    assert not os.path.exists(tmp_path / "out" / "checkpoint")


def test_skipped_steps_are_counted_between_log_steps(tmp_path, monkeypatch):
    """A step skipped for a non-finite gradient is counted even when it is not a logging step."""
    from uttt_b200.train.engine import TrainEngine
    job, model = _write(tmp_path)
    real = TrainEngine.train_step
    calls = {"n": 0}

    def flaky(self, batch):
        loss = real(self, batch)
        calls["n"] += 1
        if calls["n"] in (2, 3):                        # steps 2 and 3 report "skipped"; only step 4 logs
            self.last_stats["skipped"] = torch.tensor(True)
        return loss
    monkeypatch.setattr(TrainEngine, "train_step", flaky)
    state = lm_trainer.main(JobConfig().parse_args(["--job.config_file", job, "--model.config", model,
                                                    "--training.steps", "4", "--metrics.log_freq", "4",
                                                    "--checkpoint.interval", "100"]))
    assert state.skipped_step == 2


def test_a_failed_kernel_status_stops_training_and_saving(tmp_path, monkeypatch):
    from uttt_b200.train.engine import KernelStatusError, TrainEngine
    job, model = _write(tmp_path)
    monkeypatch.setattr(TrainEngine, "kernel_status", lambda self: 24 if self.step >= 2 else 0)
    with pytest.raises(KernelStatusError):
        lm_trainer.main(JobConfig().parse_args(["--job.config_file", job, "--model.config", model]))
    ckpt_dir = tmp_path / "out" / "checkpoint"
    assert not os.path.exists(ckpt_dir) or os.listdir(ckpt_dir) == []      # nothing was saved at the failing step
