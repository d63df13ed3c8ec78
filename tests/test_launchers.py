"""Launcher command construction, environment validation, and a fake ``torchrun`` on PATH."""
import os
import stat
import subprocess
import sys

import pytest

from uttt_b200.launch import LaunchError, build_command, main, rendezvous_args

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _files(tmp_path):
    job, model, cfg = tmp_path / "job.toml", tmp_path / "m.json", tmp_path / "c.yaml"
    for f in (job, model, cfg):
        f.write_text("x")
    return str(job), str(model), str(cfg)


def test_standalone_command(tmp_path):
    job, model, cfg = _files(tmp_path)
    cmd, dry = build_command(["lm", "--dry-run", job, model, "myrun", "--training.steps", "5"], {"NPROC_PER_NODE": "2"})
    assert dry and cmd[0] == "torchrun" and "--standalone" in cmd and "--nproc_per_node=2" in cmd
    assert cmd[cmd.index("--job.dump_folder") + 1] == "runs/myrun" and cmd[-2:] == ["--training.steps", "5"]
    cmd, _ = build_command(["nvs", cfg, "-s", "training.lr", "1e-4"], {})
    assert "uttt_b200.nvs.trainer" in cmd and cmd[-3:] == ["-s", "training.lr", "1e-4"] and "--nproc_per_node=8" in cmd


def test_multinode_arguments():
    env = {"NPROC_PER_NODE": "8", "MASTER_PORT": "29500", "MASTER_ADDR": "10.0.0.1", "WORLD_SIZE": "16",
           "NODE_RANK": "1", "JOB_UUID": "abc"}
    args, nproc = rendezvous_args(env, "x")
    assert "--nnodes=2" in args and "--node-rank=1" in args and "--rdzv-id=abc" in args
    assert "--rdzv-endpoint=10.0.0.1:29500" in args and nproc == 8


@pytest.mark.parametrize("env", [
    {"NPROC_PER_NODE": "0"}, {"NPROC_PER_NODE": "x"}, {"MASTER_ADDR": "h"}, {"WORLD_SIZE": "8"},
    {"MASTER_PORT": "29500"}, {"MASTER_PORT": "70000", "MASTER_ADDR": "h", "WORLD_SIZE": "8"},
    {"MASTER_PORT": "29500", "MASTER_ADDR": "h", "WORLD_SIZE": "12", "NPROC_PER_NODE": "8"},
    {"MASTER_PORT": "29500", "MASTER_ADDR": "h", "WORLD_SIZE": "16", "NPROC_PER_NODE": "8"},
    {"MASTER_PORT": "29500", "MASTER_ADDR": "h", "WORLD_SIZE": "16", "NPROC_PER_NODE": "8", "NODE_RANK": "2"},
])
def test_invalid_environments(env):
    with pytest.raises(LaunchError):
        rendezvous_args(env, "x")


def test_missing_config_and_unknown_kind(tmp_path):
    assert main(["lm", "--dry-run", "nope.toml", "nope.json"], {}) == 2
    assert main(["what"], {}) == 2


def test_fake_torchrun_receives_argv_and_exit_code_propagates(tmp_path):
    job, model, _ = _files(tmp_path)
    fake = tmp_path / "bin"
    fake.mkdir()
    script = fake / "torchrun"
    script.write_text("#!/bin/sh\nprintf '%s\\n' \"$@\" > \"$FAKE_OUT\"\nexit 7\n")
    script.chmod(script.stat().st_mode | stat.S_IEXEC)
    env = dict(os.environ, PATH=f"{fake}:{os.environ['PATH']}", FAKE_OUT=str(tmp_path / "argv.txt"),
               NPROC_PER_NODE="1", PYTHONPATH=ROOT)
    for k in ("MASTER_ADDR", "MASTER_PORT", "WORLD_SIZE", "RANK", "NODE_RANK"):
        env.pop(k, None)
    rc = subprocess.call(["bash", os.path.join(ROOT, "launch", "train_lm.sh"), job, model], env=env,
                         stdout=subprocess.DEVNULL)
    assert rc == 7
    argv = (tmp_path / "argv.txt").read_text().split("\n")
    assert "--standalone" in argv and "uttt_b200.train.lm_trainer" in argv
    # a failing NODE_SYNC stops the launch before torchrun
    os.remove(tmp_path / "argv.txt")
    rc = subprocess.call(["bash", os.path.join(ROOT, "launch", "train_lm.sh"), job, model],
                         env=dict(env, NODE_SYNC="exit 3"), stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    assert rc == 3 and not (tmp_path / "argv.txt").exists()


def test_dataset_registry_is_forwarded_before_the_user_flags(tmp_path):
    job, model, _ = _files(tmp_path)
    reg = tmp_path / "datasets.yaml"
    reg.write_text("train:\n  files: /data/shards/data-*.arrow\nptl:\n  files: /data/books/*.arrow\n")
    env = {"NPROC_PER_NODE": "1", "UTTT_LM_DATASETS": str(reg)}
    cmd, _ = build_command(["lm", job, model, "--training.data_files", "/mine/*.arrow"], env)
    first = cmd.index("--training.data_files")
    assert cmd[first + 1] == "/data/shards/data-*.arrow" and cmd[-2:] == ["--training.data_files", "/mine/*.arrow"]
    reg.write_text("train:\n  files: PATH/TO/long-data-collections-arrow/data-*.arrow\n")
    with pytest.raises(LaunchError, match="placeholder"):
        build_command(["lm", job, model], env)
    reg.write_text("train: {}\n")
    with pytest.raises(LaunchError, match="train.files"):
        build_command(["lm", job, model], env)
    cmd, _ = build_command(["lm", job, model], {"NPROC_PER_NODE": "1", "UTTT_LM_DATASETS": str(tmp_path / "absent.yaml")})
    assert "--training.data_files" not in cmd


def test_view_synthesis_dataset_registry(tmp_path):
    import yaml
    from uttt_b200.nvs.trainer import resolve_datasets
    reg = tmp_path / "datasets.yaml"
    reg.write_text(yaml.safe_dump({"obj": {"train": "/m/train.txt", "eval": "/m/eval.txt"},
                                   "dl3dv": {"train": "PATH/TO/dl3dv_train_manifest.txt", "eval": "/m/e.txt"}}))

    def cfg(**tr):
        return {"training": dict(tr)}

    out = resolve_datasets(cfg(dataset="obj"), str(reg))
    assert out["training"]["dataset_path"] == "/m/train.txt" and out["eval_dataset_path"] == "/m/eval.txt"
    out = resolve_datasets(cfg(dataset="obj", dataset_path="/mine.txt"), str(reg))            # the configuration wins
    assert out["training"]["dataset_path"] == "/mine.txt" and out["eval_dataset_path"] == "/m/eval.txt"
    out = resolve_datasets(cfg(dataset="obj", dataset_path="PATH/TO/x.txt", dataset_registry=str(reg)))
    assert out["training"]["dataset_path"] == "/m/train.txt"                                   # a placeholder does not
    with pytest.raises(ValueError, match="placeholder"):
        resolve_datasets(cfg(dataset="dl3dv"), str(reg))
    with pytest.raises(KeyError, match="Available"):
        resolve_datasets(cfg(dataset="re10k"), str(reg))
    with pytest.raises(FileNotFoundError, match="datasets.example.yaml"):
        resolve_datasets(cfg(dataset="obj"), str(tmp_path / "none.yaml"))
    assert "dataset_path" not in resolve_datasets(cfg(dataset="synthetic"), str(tmp_path / "none.yaml"))["training"]
    example = yaml.safe_load(open(os.path.join(ROOT, "configs", "nvs", "datasets.example.yaml")))
    assert set(example) == {"obj", "dl3dv"} and all(set(v) == {"train", "eval"} for v in example.values())
