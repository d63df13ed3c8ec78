"""View-synthesis trainer.

    torchrun -m uttt_b200.nvs.trainer --config cfg.yaml [-s dotted.key value ...] [--load PATH]

Same job semantics as the reference script (uttt_nvs/train/trainer.py:44-814): one YAML per run with ``-s``
overrides (values parsed with ``literal_eval``; ``block.x`` is an alias of ``model.block_config.params.x``),
a ``datasets.yaml`` registry keyed by ``training.dataset``, a global-batch guard
(``batch_size_per_gpu * world * grad_accum_steps == total_batch_size``), bf16 compute, AdamW with decay on
tensors of rank >= 2, warmup + cosine schedule, a collective finite-loss vote before every backward,
gradient clipping with outlier-step skipping, atomic ``ckpt_<step>.pt`` checkpoints with retention and
resume, and a ``[TRAIN_SUMMARY]`` line with the average step time and peak memory.  Also as there: the pass budget
``max_fwdbwd_passes x grad_accum_steps`` rounded up to whole epochs unless ``round_max_fwdbwd_passes_to_epoch`` is off
(:func:`job_overview`), squared-error-only warm-up for ``l2_warmup_steps`` passes, in-training evaluation every
``eval_every`` passes (and after the first pass unless ``eval_first_step`` is off) on ``eval_dataset_path`` with
``eval_num_views`` views, visuals every ``vis_every`` passes, metrics every ``wandb_log_every`` passes
(``metrics.jsonl`` in the run folder; Weights & Biases too when the package and a key are present).

Data parallelism runs through :class:`uttt_b200.parallel.fsdp.ShardedTrainer`: gradients are reduced and
AdamW is applied on per-rank shards by the fused peer-memory kernels (the role DDP's bucketed all-reduce
plus a fused optimizer play in the reference).
"""
from __future__ import annotations

import argparse
import ast
import math
import os
import sys
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import yaml

from ..parallel.fsdp import AdamWConfig, ShardedTrainer
from ..train.engine import init_distributed
from .checkpoint import checkpoint_job, delete_previous_job, resume_job, select_resume_path
from .data import NVSDataset, ResumableDistributedSampler, SyntheticScenes
from .model import LVSMModel, get_obj_by_name, resolve_model_class

ALIASES = {"block.": "model.block_config.params.", "block0.": "model.block_config.0.params.",
           "block1.": "model.block_config.1.params.", "block2.": "model.block_config.2.params."}


def apply_overrides(cfg: Dict[str, Any], pairs: List[List[str]]) -> Dict[str, Any]:
    for key, raw in pairs:
        for short, full in ALIASES.items():
            if key.startswith(short):
                key = full + key[len(short):]
        try:
            value = ast.literal_eval(raw)
        except (ValueError, SyntaxError):
            value = raw
        node = cfg
        parts = [int(p) if p.lstrip("-").isdigit() else p for p in key.split(".")]     # integers index lists
        for p in parts[:-1]:
            if isinstance(node, dict) and p not in node:
                node[p] = {}
            node = node[p]
        node[parts[-1]] = value
    return cfg


DATASET_REGISTRY = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "configs",
                                "nvs", "datasets.yaml")


def resolve_datasets(cfg: Dict[str, Any], registry_path: Optional[str] = None) -> Dict[str, Any]:
    """``training.dataset: obj | dl3dv | ...`` selects a block ``{train: manifest, eval: manifest}`` of the dataset
    registry (``training.dataset_registry``, default ``configs/nvs/datasets.yaml``, a filled-in copy of
    ``datasets.example.yaml``).  A path written in the configuration wins over the registry; a registry that is
    missing, lacks the block or still holds ``PATH/TO/`` placeholders is an error
    (uttt_nvs/train/trainer.py:153-196).  ``dataset: synthetic`` (or none) needs no registry."""
    tr = cfg.setdefault("training", {})
    name = tr.get("dataset")
    if not name or name == "synthetic":
        return cfg
    reg_path = registry_path or tr.get("dataset_registry") or DATASET_REGISTRY

    def unset(v) -> bool:
        return not v or str(v).startswith("PATH/TO/")

    if not os.path.exists(reg_path):
        if not unset(tr.get("dataset_path")):
            return cfg                                # the configuration names its manifests itself
        raise FileNotFoundError(f"Dataset registry '{reg_path}' not found. Copy configs/nvs/datasets.example.yaml to "
                                f"configs/nvs/datasets.yaml and fill in your manifest paths, or set "
                                f"training.dataset_path explicitly.")
    with open(reg_path) as fh:
        reg = yaml.safe_load(fh) or {}
    if name not in reg:
        raise KeyError(f"Dataset '{name}' is not defined in {reg_path}. Available: {sorted(reg)}")
    for field, holder, key in (("train", tr, "dataset_path"), ("eval", cfg, "eval_dataset_path")):
        value = (reg[name] or {}).get(field)
        if not unset(holder.get(key)):
            continue
        if unset(value):
            raise ValueError(f"`{name}.{field}` in {reg_path} still holds its placeholder value. Point it at a "
                             f"manifest (python -m uttt_b200.nvs.manifests build ...).")
        holder[key] = value
    return cfg


def load_config(path: str, overrides: Optional[List[List[str]]] = None, datasets_yaml: Optional[str] = None):
    with open(path) as fh:
        cfg = yaml.safe_load(fh)
    cfg = apply_overrides(cfg, overrides or [])
    return resolve_datasets(cfg, datasets_yaml)


def check_batch_arithmetic(cfg: Dict[str, Any], world: int) -> int:
    tr = cfg["training"]
    accum = int(tr.get("grad_accum_steps", 1))
    got = int(tr["batch_size_per_gpu"]) * world * accum
    want = int(tr.get("total_batch_size", got))
    if got != want:
        raise ValueError(f"batch_size_per_gpu ({tr['batch_size_per_gpu']}) x world ({world}) x grad_accum_steps "
                         f"({accum}) = {got} != total_batch_size ({want})")
    return accum


def job_overview(num_gpus: int, num_train_samples: int, batch_size_per_gpu: int, grad_accum_steps: int,
                 max_fwdbwd_passes: int = int(1e10), round_max_fwdbwd_passes_to_epoch: bool = True) -> Dict[str, int]:
    """Sizes of a run (uttt_nvs/train/checkpoint.py:213-255).  ``max_fwdbwd_passes`` is the budget in passes; with
    rounding the run ends on an epoch boundary after it (always at least one more partial epoch's worth)."""
    per_pass = batch_size_per_gpu * num_gpus
    per_epoch = max(1, int(num_train_samples / per_pass))
    if round_max_fwdbwd_passes_to_epoch:
        epochs = int(max_fwdbwd_passes / per_epoch) + 1
        passes = per_epoch * epochs
    else:
        passes = max_fwdbwd_passes
        epochs = (passes + per_epoch - 1) // per_epoch
    return {"batch_size_per_fwdbwd_pass": per_pass, "batch_size_per_param_update": per_pass * grad_accum_steps,
            "num_fwdbwd_passes_per_epoch": per_epoch, "num_param_updates_per_epoch": int(per_epoch / grad_accum_steps),
            "num_fwdbwd_passes": passes, "num_param_updates": (passes + grad_accum_steps - 1) // grad_accum_steps,
            "num_epochs": epochs}


class MetricsLog:
    """Rank 0's metric sink: one JSON object per line in ``<run>/metrics.jsonl``; mirrored to Weights & Biases when the
    package is importable and a key is available (``WANDB_API_KEY`` or ``wandb:`` in ``training.api_key_path``).
    The run id is kept in ``wandb_id.txt`` so that a resumed job continues the same run."""

    def __init__(self, out_dir: str, cfg: Dict[str, Any], enabled: bool):
        self.path, self.run = None, None
        if not enabled:
            return
        self.path = os.path.join(out_dir, "metrics.jsonl")           # the folder is made by the first line written
        tr = cfg.get("training", {})
        key = os.environ.get("WANDB_API_KEY", "")
        key_file = tr.get("api_key_path")
        if not key and key_file and os.path.exists(str(key_file)):
            with open(key_file) as fh:
                key = str((yaml.safe_load(fh) or {}).get("wandb", "") or "")
        if not key or key.startswith("YOUR_"):
            return
        try:
            import wandb
        except ImportError:
            print("wandb is not installed: metrics go to metrics.jsonl only", flush=True)
            return
        os.environ.setdefault("WANDB_API_KEY", key)
        if tr.get("wandb_offline", False):
            os.environ["WANDB_MODE"] = "offline"
        os.makedirs(out_dir, exist_ok=True)
        id_file = os.path.join(out_dir, "wandb_id.txt")
        run_id = open(id_file).read().strip() if os.path.exists(id_file) else None
        self.run = wandb.init(project=os.environ.get("WANDB_PROJECT", "uttt-nvs"), name=cfg.get("exp_name", "run"),
                              dir=os.path.join(out_dir, "wandb"), id=run_id, resume=tr.get("wandb_resume", "allow"),
                              config=cfg)
        if run_id is None:
            with open(id_file, "w") as fh:
                fh.write(self.run.id)

    def log(self, payload: Dict[str, Any], step: int, images: Optional[Dict[str, Any]] = None) -> None:
        if self.path is None:
            return
        import json
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        with open(self.path, "a") as fh:
            fh.write(json.dumps({"step": step, **payload}) + "\n")
        if self.run is not None:
            import wandb
            extra = {k: wandb.Image(v) for k, v in (images or {}).items()}
            self.run.log({**payload, **extra}, step=step)


def lr_at(step: int, base: float, warmup: int, total: int, kind: str = "cosine", init_ratio: float = 0.0) -> float:
    """Learning rate of optimizer step number ``step`` (0-based): linear warm-up from ``init_ratio x base`` over
    ``warmup`` steps (so the very first step runs at ``init_ratio x base``, zero by default), then cosine / linear
    decay to zero at ``total`` or constant (uttt_nvs/train/optimizer.py:53-112)."""
    if kind not in ("cosine", "linear", "constant"):
        raise ValueError(f"Not support LR scheduler type {kind}.")
    if not 0.0 <= init_ratio <= 1.0:
        raise ValueError("warmup_init_ratio must be in [0, 1].")
    if warmup > 0 and step < warmup:
        return base * (init_ratio + (1.0 - init_ratio) * step / max(warmup, 1))
    if kind == "constant" or total <= warmup:
        return base
    if kind == "linear":
        return base * max(0.0, (total - step) / max(total - warmup, 1))
    prog = min(max((step - warmup) / max(total - warmup, 1), 0.0), 1.0)
    return base * 0.5 * (1.0 + math.cos(math.pi * prog))


class _OptimizerView:
    """state_dict()/load_state_dict() adapters so the checkpoint file keeps the reference's top-level keys.

    Two layouts are read: this package's (fp32 master and moments by parameter name) and ``torch.optim.AdamW``'s as
    the reference writes it (``state`` by index over two groups: parameters of rank >= 2 in ``named_parameters``
    order, then the rest; uttt_nvs/train/optimizer.py:15-50).  From the latter the moments and the step count are
    taken and the fp32 masters come from the checkpoint's own fp32 weights (``model_state``)."""

    def __init__(self, trainer: ShardedTrainer, model: Optional[torch.nn.Module] = None):
        self.trainer, self.model = trainer, model
        self.loaded = False          # True once fp32 masters and moments came from a checkpoint

    def _groups(self):
        named = [(n, p) for n, p in self.model.named_parameters() if p.requires_grad]
        return [[n for n, p in named if p.dim() >= 2], [n for n, p in named if p.dim() < 2]]

    def state_dict(self):
        """The moments in ``torch.optim.AdamW``'s layout (what the reference's trainer writes and reads), so that a
        run can move between the two implementations in either direction.  ``self.masters`` afterwards holds the
        fp32 weights by name: the checkpoint stores those as the model's values."""
        own = self.trainer.optimizer_state_dict()
        cfg = self.trainer.opt
        self.masters = {n: st["master"] for n, st in own["state"].items() if "master" in st}
        if self.model is None:
            return own
        state, groups, idx = {}, [], 0
        step = torch.tensor(float(own["step"]))
        for names, decay in zip(self._groups(), (float(cfg.weight_decay), 0.0)):
            ids = []
            for name in names:
                st = own["state"].get(name)
                if st is not None and "exp_avg" in st:
                    state[idx] = {"step": step.clone(), "exp_avg": st["exp_avg"], "exp_avg_sq": st["exp_avg_sq"]}
                ids.append(idx)
                idx += 1
            groups.append({"lr": float(getattr(self, "last_lr", cfg.lr)), "initial_lr": float(cfg.lr),
                           "betas": (float(cfg.beta1), float(cfg.beta2)), "eps": float(cfg.eps), "weight_decay": decay,
                           "amsgrad": False, "maximize": False, "foreach": None, "capturable": False,
                           "differentiable": False, "fused": None, "params": ids})
        return {"state": state, "param_groups": groups, "skipped_steps": own.get("skipped_steps", 0)}

    def _from_torch_adamw(self, sd, model_state):
        named = [(n, p) for n, p in self.model.named_parameters() if p.requires_grad]
        groups = [[n for n, p in named if p.dim() >= 2], [n for n, p in named if p.dim() < 2]]
        if len(sd["param_groups"]) != 2 or [len(g["params"]) for g in sd["param_groups"]] != [len(g) for g in groups]:
            raise ValueError("optimizer param groups do not match this model (decay: rank >= 2, no decay: the rest)")
        shapes = dict((n, tuple(p.shape)) for n, p in named)
        state, step = {}, 0
        for group, names in zip(sd["param_groups"], groups):
            for idx, name in zip(group["params"], names):
                entry = sd["state"].get(idx)
                if entry is None:
                    continue
                if tuple(entry["exp_avg"].shape) != shapes[name]:
                    raise ValueError(f"optimizer state of {name} has shape {tuple(entry['exp_avg'].shape)}, "
                                     f"expected {shapes[name]}")
                state[name] = {"exp_avg": entry["exp_avg"].float(), "exp_avg_sq": entry["exp_avg_sq"].float()}
                if model_state is not None and name in model_state:
                    state[name]["master"] = model_state[name].float()
                step = max(step, int(entry["step"]))
        return {"step": step, "skipped_steps": int(sd.get("skipped_steps", 0)), "state": state}

    def load_state_dict(self, sd, model_state=None):
        if "param_groups" in sd:
            sd = self._from_torch_adamw(sd, model_state)
        self.trainer.load_optimizer_state_dict(sd)
        self.loaded = True


class _Schedule:
    """Counter of optimizer steps, stored with the keys of a ``torch.optim.lr_scheduler.LambdaLR`` state."""

    def __init__(self, base_lr: float = 0.0):
        self.step_count, self.base_lr, self.last_lr = 0, base_lr, base_lr

    def state_dict(self):
        return {"base_lrs": [self.base_lr, self.base_lr], "last_epoch": self.step_count,
                "_step_count": self.step_count + 1, "_last_lr": [self.last_lr, self.last_lr],
                "_get_lr_called_within_step": False, "lr_lambdas": [None, None], "step_count": self.step_count}

    def load_state_dict(self, sd):
        self.step_count = int(sd.get("step_count", sd.get("last_epoch", 0)))


class NVSTrainer:
    def __init__(self, cfg: Dict[str, Any], device: Optional[torch.device] = None, load: str = ""):
        self.cfg = cfg
        self.rank, self.world, local = init_distributed()
        self.device = device or (torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu"))
        tr = cfg["training"]
        self.accum = check_batch_arithmetic(cfg, self.world)
        if cfg["model"].get("act_ckpt"):
            raise NotImplementedError("model.act_ckpt is not supported: gradient checkpointing is already applied "
                                      "inside the blocks. Remove `act_ckpt: true` from the config.")
        torch.manual_seed(int(tr.get("seed", 0)))                  # the same initial weights on every rank
        model_cls = resolve_model_class(cfg["model"].get("class_name"))
        self.model = model_cls(cfg).to(self.device)
        import random as _random                                   # from here on every process draws its own stream
        _random.seed(int(tr.get("seed", 0)) + self.rank)
        torch.manual_seed(int(tr.get("seed", 0)) + self.rank)
        opt = AdamWConfig(lr=float(tr.get("lr", 4e-4)), beta1=float(tr.get("beta1", 0.9)),
                          beta2=float(tr.get("beta2", 0.95)), eps=1e-8, weight_decay=float(tr.get("weight_decay", 0.05)),
                          max_norm=float(tr.get("grad_clip_norm", 1.0)), skip_nan_inf=True)
        units = [(f"transformer_blocks.blocks.{i}", b) for i, b in
                 enumerate(getattr(self.model.transformer_blocks, "blocks", []))]
        self.trainer = ShardedTrainer(self.model, units, opt, no_decay=lambda n, p: p.dim() < 2)
        self.optimizer, self.schedule = _OptimizerView(self.trainer, self.model), _Schedule(float(tr.get("lr", 4e-4)))
        # the environment variable wins over the file, so one exported path redirects every configuration
        self.out_dir = os.path.join(os.environ.get("UTTT_NVS_OUT_DIR") or tr.get("out_dir", "experiments"),
                                    cfg.get("exp_name", "run"))
        self.fwdbwd_step = 0
        self.update_step = 0
        resume = select_resume_path(self.out_dir, load, tr.get("load", "") or "")
        if resume:
            # a run continued from its own folder keeps its counters whatever the file says; weights brought in from
            # elsewhere may start the counters (and, unless asked otherwise, the optimizer) afresh
            reset = (bool(tr.get("reset_training_state", False)) and resume != self.out_dir) \
                or bool(tr.get("force_reset_training_state", False))
            _, _, self.fwdbwd_step, self.update_step = resume_job(
                resume, self.model, self.optimizer, self.schedule, reset_training_state=reset,
                load_optimizer_state_when_reset_training_state=bool(
                    tr.get("load_optimizer_state_when_reset_training_state", False)) and reset)
            if not self.optimizer.loaded:
                # only the model came back (a reset of the training state): rebuild the fp32 masters from it.
                # With optimizer state loaded the masters are already exact; re-reading the bf16 compute copy
                # would round them.
                self.trainer.load_model_state()
        self.num_train_samples: Optional[int] = None               # None: the synthetic stream has no epochs
        self.data = self._build_data()
        budget = int(tr.get("max_fwdbwd_passes", int(1e10))) * self.accum
        if self.num_train_samples is None:
            self.overview = {"num_fwdbwd_passes": int(tr.get("max_fwdbwd_passes", 20000)),
                             "num_fwdbwd_passes_per_epoch": int(tr.get("max_fwdbwd_passes", 20000)),
                             "num_param_updates": max(int(tr.get("max_fwdbwd_passes", 20000)) // self.accum, 1)}
        else:
            self.overview = job_overview(self.world, self.num_train_samples, int(tr["batch_size_per_gpu"]), self.accum,
                                         budget, bool(tr.get("round_max_fwdbwd_passes_to_epoch", True)))
        self.total = self.overview["num_fwdbwd_passes"]
        self.start_step = self.fwdbwd_step
        self.metrics = MetricsLog(self.out_dir, cfg, enabled=self.rank == 0 and bool(tr.get("log_metrics", True)))
        self._eval_data = None
        self.step_times: List[float] = []
        self._graphs: Dict[Any, Any] = {}
        self._passes_run = 0                       # of this process (a resumed run also warms up before a capture)
        self.graph_error: Optional[str] = None

    def _build_data(self):
        tr = self.cfg["training"]
        size = self.cfg["model"]["image_size"]
        size = size if isinstance(size, int) else size[0]
        if tr.get("dataset", "synthetic") == "synthetic" or not tr.get("dataset_path"):
            src = SyntheticScenes(int(tr["batch_size_per_gpu"]), int(tr.get("num_views", 6)), size,
                                  seed=int(tr.get("seed", 0)), rank=self.rank)
            src.step = self.fwdbwd_step
            return iter(src)
        ds = NVSDataset(tr["dataset_path"], int(tr.get("num_views", 12)), size, tr.get("max_num_objects"))
        self.num_train_samples = len(ds)
        sampler = ResumableDistributedSampler(ds, num_replicas=self.world, rank=self.rank, shuffle=True, seed=0,
                                              drop_last=True)
        if len(sampler) < int(tr["batch_size_per_gpu"]):
            raise ValueError(f"zero complete batches: {len(ds)} manifest entries over {self.world} process(es) give "
                             f"{len(sampler)} samples per process, fewer than batch_size_per_gpu="
                             f"{tr['batch_size_per_gpu']}; repeat the manifest entries or lower the batch size")
        per_epoch = max(len(sampler) // int(tr["batch_size_per_gpu"]), 1)
        sampler.set_epoch(self.fwdbwd_step // per_epoch)
        sampler.set_resume_offset((self.fwdbwd_step % per_epoch) * int(tr["batch_size_per_gpu"]))
        loader = torch.utils.data.DataLoader(ds, batch_size=int(tr["batch_size_per_gpu"]), sampler=sampler,
                                             num_workers=int(tr.get("num_workers", 0)), drop_last=True,
                                             pin_memory=torch.cuda.is_available(),
                                             **self._worker_options(int(tr.get("num_workers", 0))))

        def forever():
            epoch = self.fwdbwd_step // per_epoch
            while True:
                for batch in loader:
                    yield batch
                epoch += 1
                sampler.set_epoch(epoch)
        return forever()

    def _worker_options(self, workers: int) -> Dict[str, Any]:
        pf = self.cfg["training"].get("prefetch_factor")
        return {"prefetch_factor": int(pf), "persistent_workers": True} if workers > 0 and pf else {}

    def train_pass(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        """One forward/backward pass; an optimizer step every ``grad_accum_steps`` passes."""
        tr = self.cfg["training"]
        t0 = time.time()
        batch = {k: v.to(self.device, non_blocking=True) for k, v in batch.items() if torch.is_tensor(v)}
        self.model.train()
        warm = self.fwdbwd_step < int(tr.get("l2_warmup_steps", 0))
        if warm != self.model._l2_only:
            self.model.l2_warmup(warm)
            self.release_graphs()                             # a captured pass has the loss terms baked in
        loss, psnr, vote = self._forward_backward(batch)
        self.fwdbwd_step += 1
        stats: Dict[str, Any] = {"loss": loss, "psnr": psnr, "finite": vote}
        if self.accum > 1:
            self.trainer.accumulate_micro_batch()             # every pass, the last one included
        if self.fwdbwd_step % self.accum == 0 or self.fwdbwd_step == self.total:
            lr = lr_at(self.update_step, float(tr.get("lr", 4e-4)), int(tr.get("warmup", 0)),
                       self.overview["num_param_updates"], tr.get("scheduler_type", "cosine"),
                       float(tr.get("warmup_init_ratio", 0.0)))
            skip_above = None
            clip = float(tr.get("grad_clip_norm", 1.0))
            if clip > 0 and self.fwdbwd_step > int(tr.get("may_skip_gradnorm_after", 0)):
                skip_above = float(tr.get("allowed_gradnorm_factor", 5)) * clip
            out = self.trainer.step(lr=lr, skip_above=skip_above)
            self.update_step += 1
            self.schedule.step_count = self.update_step
            self.schedule.last_lr = self.optimizer.last_lr = lr
            stats.update(grad_norm=out["grad_norm"], skipped=out["skipped"], lr=lr)
        self.step_times.append(time.time() - t0)
        return stats

    def _forward_backward_eager(self, batch):
        result = self.model(batch)
        loss = result["loss_metrics"]["loss"]
        vote = torch.isfinite(loss.detach()).float()
        if self.world > 1 and not (vote.is_cuda and torch.cuda.is_current_stream_capturing()):
            # every rank skips together.  A captured graph holds no collective: there a non-finite loss leaves
            # non-finite gradients, and the optimizer's own all-reduced norm check skips the step on every rank.
            dist.all_reduce(vote, op=dist.ReduceOp.MIN)
        (loss * vote / self.accum).backward()
        return loss.detach(), result["loss_metrics"]["psnr"], vote

    def _forward_backward(self, batch):
        """Eager, or (``training.cuda_graph``) replayed from a graph captured on the third pass with these input
        shapes: a pass is tens of thousands of small launches, which keep the host busier than the device."""
        tr = self.cfg["training"]
        use_graph = (bool(tr.get("cuda_graph", False)) and self.device.type == "cuda" and self.graph_error is None
                     and self._passes_run >= 2)
        self._passes_run += 1
        if not use_graph:
            return self._forward_backward_eager(batch)
        key = tuple((k, tuple(v.shape), v.dtype) for k, v in sorted(batch.items()))
        entry = self._graphs.get(key)
        if entry is None:
            try:
                torch.cuda.synchronize(self.device)
                torch.cuda.empty_cache()
                static = {k: v.clone() for k, v in batch.items()}
                graph = torch.cuda.CUDAGraph()
                from ..ops import functional as F
                before = F.launch_count()
                with torch.cuda.graph(graph):
                    outs = self._forward_backward_eager(static)
                entry = (graph, static, outs, F.launch_count() - before)
            except Exception as exc:                      # capture refused an operation: stay eager from here on
                self.graph_error = f"{type(exc).__name__}: {exc}"
                return self._forward_backward_eager(batch)
            self._graphs[key] = entry
        graph, static, outs, launches = entry
        for k, v in batch.items():
            static[k].copy_(v)
        graph.replay()
        from ..ops import functional as F
        F._count(launches)
        return outs

    def release_graphs(self) -> None:
        self._graphs.clear()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()

    def save(self) -> Optional[str]:
        """``ckpt_<pass:016>.pt`` in the reference's format: fp32 weights under the model's parameter names, the
        moments as a ``torch.optim.AdamW`` state over (rank >= 2 | rest) groups, a ``LambdaLR``-style schedule state
        and the two counters."""
        tr = self.cfg["training"]
        opt_sd = self.optimizer.state_dict()          # collective
        masters = getattr(self.optimizer, "masters", {})
        path = None
        if self.rank == 0:
            class _Frozen:
                def state_dict(_self):
                    return opt_sd

            class _FullPrecision:
                """The model's state with the optimizer's fp32 masters in place of the bf16 compute copies."""
                def state_dict(_self):
                    sd = self.model.state_dict()
                    return {k: (masters[k].reshape(v.shape) if k in masters else v) for k, v in sd.items()}
            path = checkpoint_job(self.out_dir, _FullPrecision(), _Frozen(), self.schedule, self.fwdbwd_step,
                                  self.update_step)
            delete_previous_job(self.out_dir, self.fwdbwd_step, int(tr.get("save_last_n_ckpts", 3)))
        if self.world > 1:
            dist.barrier()
        return path

    # ------------------------------------------------------------------ in-training evaluation and visuals
    def _build_eval(self):
        """(iterator factory, number of batches per evaluation).  Real data: ``eval_dataset_path`` with
        ``eval_num_views`` views, epoch 0 of a sharded sampler every time; synthetic data: a fixed-seed stream."""
        tr = self.cfg["training"]
        bs = int(tr["batch_size_per_gpu"])
        views = int(tr.get("eval_num_views", tr.get("num_views", 12)))
        size = self.cfg["model"]["image_size"]
        size = size if isinstance(size, int) else size[0]
        steps = min(511 // bs // self.world + 1, 8)
        if self.num_train_samples is None:
            return (lambda: iter(SyntheticScenes(bs, views, size, seed=9595, rank=self.rank))), steps
        path = self.cfg.get("eval_dataset_path")
        if not path or str(path).startswith("PATH/TO/"):
            raise ValueError("`eval_dataset_path` still holds its placeholder value. Point it at an evaluation "
                             "manifest (python -m uttt_b200.nvs.manifests build ...), or switch the in-training "
                             "evaluation off with `-s training.eval_every 0`.")
        ds = NVSDataset(path, views, size)
        available = len(ds) // self.world // bs
        if available < 1:
            raise ValueError(
                f"In-training evaluation cannot run: {len(ds)} evaluation scenes split over {self.world} ranks at "
                f"{bs} per rank leaves some ranks with no batch at all.\nDisable it with `-s training.eval_every 0` and "
                f"evaluate separately with `python -m uttt_b200.nvs.eval.evaluate`, or run on at most "
                f"{max(len(ds) // bs, 1)} ranks.")
        sampler = ResumableDistributedSampler(ds, num_replicas=self.world, rank=self.rank, shuffle=True, seed=0,
                                              drop_last=True)
        loader = torch.utils.data.DataLoader(ds, batch_size=bs, sampler=sampler, drop_last=True,
                                             num_workers=int(tr.get("num_workers", 0)),
                                             pin_memory=torch.cuda.is_available())

        def fresh():
            sampler.set_epoch(0)
            return iter(loader)
        return fresh, max(min(steps, available), 1)

    def _avg(self, t: torch.Tensor) -> torch.Tensor:
        t = t.detach().float().clone()
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            t /= self.world
        return t

    @torch.no_grad()
    def evaluate(self) -> Dict[str, float]:
        """Mean loss / PSNR / per-view PSNR / expert-frequency extrema over the evaluation batches and ranks; visuals
        of the last batch in ``eval_<pass>/``."""
        if self._eval_data is None:
            self._eval_data = self._build_eval()
        fresh, steps = self._eval_data
        if self.rank == 0:
            print(f"Evaluating at iter {self.fwdbwd_step} eval_steps {steps}", flush=True)
        was_warm = self.model._l2_only
        self.model.eval()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()
        it = fresh()
        sums: Dict[str, torch.Tensor] = {}
        result = batch = None
        for _ in range(steps):
            batch = {k: v.to(self.device, non_blocking=True) for k, v in next(it).items() if torch.is_tensor(v)}
            result = self.model(batch)
            for key in ("loss", "psnr", "psnr_loc", "moe_freq_max", "moe_freq_min"):
                if key in result["loss_metrics"]:
                    v = result["loss_metrics"][key].detach().float() / steps
                    sums[key] = v if key not in sums else sums[key] + v
        result["loss_metrics"]["psnr_loc"] = self._avg(result["loss_metrics"]["psnr_loc"])
        images = None
        if self.rank == 0:
            images = self.model.save_visuals(os.path.join(self.out_dir, f"eval_{self.fwdbwd_step:08d}"), result, batch)
        out: Dict[str, float] = {}
        for key, v in sums.items():
            v = self._avg(v)
            if key.endswith("_loc"):
                out.update({f"{key}_{i:03}": float(x) for i, x in enumerate(v)})
            else:
                out[key] = float(v)
        payload = {**{f"eval/{k}": v for k, v in out.items() if "_loc_" not in k},
                   **{f"eval_loc/{k}": v for k, v in out.items() if "_loc_" in k}}
        self.metrics.log(payload, self.fwdbwd_step, {f"eval_{k}": v for k, v in (images or {}).items()})
        if self.rank == 0:
            print(f"eval/loss: {out['loss']}, eval/psnr: {out['psnr']} at iter {self.fwdbwd_step}", flush=True)
        if self.world > 1:
            dist.barrier()
        self.model.train()
        self.model.l2_warmup(was_warm)
        return out

    @torch.no_grad()
    def _visuals(self, batch) -> None:
        if self.rank == 0:
            batch = {k: v.to(self.device, non_blocking=True) for k, v in batch.items() if torch.is_tensor(v)}
            images = self.model.save_visuals(os.path.join(self.out_dir, f"iter_{self.fwdbwd_step:08d}"),
                                             self.model(batch), batch)
            self.metrics.log({}, self.fwdbwd_step, {f"train_{k}": v for k, v in images.items()})
        if self.world > 1:
            dist.barrier()

    def fit(self, max_passes: Optional[int] = None) -> Dict[str, float]:
        tr = self.cfg["training"]
        total = self.total if max_passes is None else min(self.total, self.fwdbwd_step + max_passes)
        eval_every = int(tr.get("eval_every", 2000))
        vis_every = int(tr.get("vis_every", 0) or 0)
        log_every = int(tr.get("wandb_log_every", 50) or 50)
        per_epoch = self.overview["num_fwdbwd_passes_per_epoch"]
        t_start = time.time()
        while self.fwdbwd_step < total:
            batch = next(self.data)
            stats = self.train_pass(batch)
            step = self.fwdbwd_step
            if self.rank == 0 and step % int(tr.get("print_every", 20)) == 0:
                print(f"epoch: {(step - 1) // per_epoch}, fwdbwd_pass_step: {step}/{per_epoch}, "
                      f"time: {self.step_times[-1]:06f}, param_update_step: {self.update_step}, "
                      f"lr: {stats.get('lr', 0):06f}\n\tloss: {float(stats['loss']):06f}, "
                      f"psnr: {float(stats['psnr']):06f}", flush=True)
            if step % log_every == 0 or step < 100 + self.start_step:
                payload = {"iter": step, "fwdbwd_pass_step": step, "param_update_step": self.update_step,
                           "lr": float(stats.get("lr", 0.0)), "iter_time": self.step_times[-1],
                           "epoch": (step - 1) // per_epoch, "train/loss": float(self._avg(stats["loss"])),
                           "train/psnr": float(self._avg(stats["psnr"]))}
                if "grad_norm" in stats:
                    payload["grad_norm"] = float(stats["grad_norm"])
                self.metrics.log(payload, step)
            if step % int(tr.get("checkpoint_every", 500)) == 0 or step == total:
                self.save()
            if vis_every > 0 and step % vis_every == 0:
                self._visuals(batch)
            if eval_every > 0 and (step % eval_every == 0 or (bool(tr.get("eval_first_step", True))
                                                              and step == self.start_step + 1)):
                self.evaluate()
        passes = max(len(self.step_times), 1)
        summary = {"avg_step_time_s": sum(self.step_times) / passes,
                   "peak_allocated_gib": torch.cuda.max_memory_allocated() / 2 ** 30 if torch.cuda.is_available() else 0.0,
                   "peak_reserved_gib": torch.cuda.max_memory_reserved() / 2 ** 30 if torch.cuda.is_available() else 0.0}
        if self.rank == 0:
            print(f"[TRAIN_SUMMARY] steps={len(self.step_times)} total_time={time.time() - t_start:.1f}s "
                  + " ".join(f"{k}={v:.4f}" for k, v in summary.items()), flush=True)
        return summary


def main(argv: Optional[List[str]] = None) -> None:
    ap = argparse.ArgumentParser(description="View-synthesis trainer")
    ap.add_argument("config_file", nargs="?", default=None, help="YAML configuration (also --config)")
    ap.add_argument("--config", default=None)
    ap.add_argument("-s", "--set", nargs=2, action="append", default=[], metavar=("KEY", "VALUE"))
    ap.add_argument("--load", default="", help="load weights from another run or file")
    ap.add_argument("--seed", type=int, default=None, help="base seed (rank is added); default training.seed or 9595")
    ap.add_argument("--debug", action="store_true", help="one pass, one evaluation batch, then stop")
    ap.add_argument("--wandb_project", default=None)
    ap.add_argument("--max-passes", type=int, default=None)
    args = ap.parse_args(argv)
    path = args.config or args.config_file
    if not path:
        ap.error("a configuration file is required")
    if args.wandb_project:
        os.environ["WANDB_PROJECT"] = args.wandb_project
    cfg = load_config(path, args.set)
    if args.seed is not None:
        cfg["training"]["seed"] = args.seed
    cfg["training"].setdefault("seed", 9595)
    trainer = NVSTrainer(cfg, load=args.load)
    if args.debug:
        if trainer._eval_data is None and int(cfg["training"].get("eval_every", 2000)) > 0:
            fresh, _ = trainer._build_eval()
            trainer._eval_data = (fresh, 1)
        trainer.fit(1)
    else:
        trainer.fit(args.max_passes)
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
