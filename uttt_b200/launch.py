"""Launcher: builds and runs the ``torchrun`` command for the language-model or view-synthesis trainer.

    python -m uttt_b200.launch lm  [--dry-run] <job.toml> <model.json> [job_name] [--section.key value ...]
    python -m uttt_b200.launch nvs [--dry-run] <config.yaml> [-s key value ...]

Environment (same contract as the reference's shell launchers, scripts/launch_common.sh:26-50,
uttt_llm/launch/train.sh:19-64, uttt_nvs/train/launch.sh:21-60): ``NPROC_PER_NODE`` (default 8) processes on
this node; a standalone single-node run unless ``MASTER_PORT`` is set, in which case ``MASTER_ADDR``,
``WORLD_SIZE`` (total processes, a multiple of ``NPROC_PER_NODE``) and ``NODE_RANK`` (or ``RANK``) select a
multi-node c10d rendezvous with id ``JOB_UUID``.  A partial distributed environment is an error.  With
``NODE_SYNC`` set, that command is run first on every node (e.g. to sync the code tree) and must succeed.
``--dry-run`` prints the working directory and the exact command and exits 0.
"""
from __future__ import annotations

import os
import re
import shlex
import subprocess
import sys
from typing import Dict, List, Optional, Tuple


class LaunchError(Exception):
    pass


def _positive_int(name: str, value: str) -> int:
    if not re.fullmatch(r"[1-9][0-9]{0,8}", value or ""):
        raise LaunchError(f"{name} must be a positive integer (at most nine digits), got '{value}'.")
    return int(value)


def rendezvous_args(env: Dict[str, str], default_id: str) -> Tuple[List[str], int]:
    nproc = _positive_int("NPROC_PER_NODE", env.get("NPROC_PER_NODE", "8"))
    port = env.get("MASTER_PORT", "")
    if port:
        if not env.get("MASTER_ADDR") or not env.get("WORLD_SIZE"):
            raise LaunchError("MASTER_PORT requires MASTER_ADDR and WORLD_SIZE (total processes).")
        if _positive_int("MASTER_PORT", port) > 65535:
            raise LaunchError("MASTER_PORT must be in 1..65535.")
        world = _positive_int("WORLD_SIZE", env["WORLD_SIZE"])
        if world % nproc:
            raise LaunchError("WORLD_SIZE must be a multiple of NPROC_PER_NODE; it counts processes, not nodes.")
        nnodes = world // nproc
        node_rank = env.get("NODE_RANK", env.get("RANK", ""))
        if node_rank == "":
            if nnodes != 1:
                raise LaunchError("Set NODE_RANK (or RANK) to this node index for a multi-node run.")
            node_rank = "0"
        if not re.fullmatch(r"0|[1-9][0-9]{0,8}", node_rank):
            raise LaunchError("NODE_RANK/RANK must be a non-negative integer.")
        if int(node_rank) >= nnodes:
            raise LaunchError(f"NODE_RANK/RANK must be less than NNODES={nnodes}.")
        rdzv_id = env.get("JOB_UUID", default_id)
        return ([f"--nnodes={nnodes}", f"--node-rank={node_rank}", f"--rdzv-id={rdzv_id}", "--rdzv-backend=c10d",
                 f"--rdzv-endpoint={env['MASTER_ADDR']}:{port}", f"--nproc_per_node={nproc}"], nproc)
    if any(env.get(k) for k in ("MASTER_ADDR", "WORLD_SIZE", "NODE_RANK", "RANK")):
        raise LaunchError("Partial distributed environment: set MASTER_PORT, MASTER_ADDR, WORLD_SIZE and NODE_RANK "
                          "together, or unset them for a standalone run.")
    return (["--standalone", "--local-addr", "127.0.0.1", f"--nproc_per_node={nproc}"], nproc)


def _readable(path: str, *fallback_dirs: str) -> str:
    for cand in (path, *[os.path.join(d, path) for d in fallback_dirs]):
        if os.path.isfile(cand) and os.access(cand, os.R_OK):
            return os.path.abspath(cand)
    raise LaunchError(f"Cannot read configuration: {path}")


def build_command(argv: List[str], env: Dict[str, str]) -> Tuple[List[str], bool]:
    if not argv or argv[0] in ("-h", "--help"):
        raise LaunchError(__doc__.split("\n\n")[1])
    kind, rest = argv[0], argv[1:]
    dry = False
    if rest and rest[0] == "--dry-run":
        dry, rest = True, rest[1:]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if kind == "lm":
        if len(rest) < 2:
            raise LaunchError("Expected <job.toml> <model.json>; use --help for usage.")
        job = _readable(rest[0], root, os.path.join(root, "configs"))
        model = _readable(rest[1], root, os.path.join(root, "configs"))
        rest = rest[2:]
        name = os.path.splitext(os.path.basename(model))[0]
        if rest and not rest[0].startswith("--"):
            name, rest = rest[0], rest[1:]
        rdzv, _ = rendezvous_args(env, "uttt-llm")
        cmd = ["torchrun", *rdzv, "-m", "uttt_b200.train.lm_trainer", "--job.config_file", job, "--job.dump_folder",
               f"runs/{name}", "--model.config", model]
        registry = env.get("UTTT_LM_DATASETS", os.path.join(root, "configs", "lm", "datasets.yaml"))
        if os.path.isfile(registry):
            # a filled-in dataset registry names the training shards once for every job file; flags given on the
            # command line come later and still win
            import yaml
            with open(registry, encoding="utf-8") as fh:
                doc = yaml.safe_load(fh)
            files = (doc.get("train") or {}).get("files") if isinstance(doc, dict) else None
            if not isinstance(files, str) or not files.strip():
                raise LaunchError(f"{registry} must contain a non-empty train.files string")
            if files.startswith("PATH/TO/"):
                raise LaunchError(f"train.files in {registry} still holds its placeholder value")
            cmd += ["--training.data_files", files]
        cmd += rest
    elif kind == "nvs":
        if len(rest) < 1:
            raise LaunchError("Expected <config.yaml>; use --help for usage.")
        cfg = _readable(rest[0], root, os.path.join(root, "configs"))
        rdzv, _ = rendezvous_args(env, "uttt-nvs")
        cmd = ["torchrun", *rdzv, "-m", "uttt_b200.nvs.trainer", "--config", cfg, *rest[1:]]
    else:
        raise LaunchError(f"unknown trainer '{kind}' (expected 'lm' or 'nvs')")
    return cmd, dry


def main(argv: Optional[List[str]] = None, env: Optional[Dict[str, str]] = None) -> int:
    env = dict(os.environ if env is None else env)
    try:
        cmd, dry = build_command(list(sys.argv[1:] if argv is None else argv), env)
    except LaunchError as exc:
        print(f"Launch error: {exc}", file=sys.stderr)
        return 2
    print(f"Working directory: {os.getcwd()}\nCommand: {' '.join(shlex.quote(c) for c in cmd)}")
    if dry:
        return 0
    sync = env.get("NODE_SYNC")
    if sync:
        rc = subprocess.call(sync, shell=True, env=env)
        if rc != 0:
            print(f"Launch error: NODE_SYNC command failed with exit code {rc}", file=sys.stderr)
            return rc
    env.setdefault("NCCL_DEBUG", "WARN")
    return subprocess.call(cmd, env=env)


if __name__ == "__main__":
    sys.exit(main())
