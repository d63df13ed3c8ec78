"""Checkpoint save / resume for the language-model trainer.

Layout (same as the reference, uttt_llm/flame/checkpoint_manager.py:312-451, 519-591 and
uttt_llm/flame/components/checkpoint.py:16-59):

``<dump_folder>/<folder>/step-<N>/`` holding either

* ``save_backend="dcp"``: a ``torch.distributed.checkpoint`` directory (``.metadata`` +
  ``__*.distcp``) with the keys ``model.*`` (reference parameter names, e.g.
  ``model.model.layers.0.attn.q_proj.weight``), ``optimizer.*``, ``lr_scheduler``,
  ``dataloader``, ``train_state``; or
* ``save_backend="rank0_model_only"``: ``model.pt`` = ``{"model": state_dict, "step": N}`` and
  ``metadata.json``.

Every save is written to ``step-<N>.tmp`` and published by an atomic rename, so a failed save
never damages the previous checkpoint; stale checkpoints beyond ``keep_latest_k`` are purged;
``load(step=-1)`` resumes from the newest readable step.  Gathering of sharded optimizer state
runs over the trainer's process group (gloo on CPU, NCCL on GPU); planning needs no extra group
because rank 0 writes the gathered state.
"""
from __future__ import annotations

import io
import json
import os
import re
import shutil
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

_STEP_RE = re.compile(r"^step-(\d+)$")


class MissingRankState(KeyError):
    """The checkpoint is readable but has no entry for this rank (not a corrupt file: never fall back silently)."""


@dataclass
class TrainState:
    """Counters and loss histories that survive a restart (components/checkpoint.py:16-59)."""
    step: int = 0
    skipped_step: int = 0
    token: int = 0
    elapsed: float = 0.0
    global_avg_losses: List[float] = field(default_factory=list)
    global_max_losses: List[float] = field(default_factory=list)
    log_steps: List[int] = field(default_factory=list)

    def state_dict(self) -> Dict[str, Any]:
        buf = io.BytesIO()
        torch.save({"avg": self.global_avg_losses, "max": self.global_max_losses, "steps": self.log_steps}, buf)
        return {"step": torch.tensor(self.step), "skipped_step": torch.tensor(self.skipped_step),
                "token": torch.tensor(self.token), "elapsed": torch.tensor(self.elapsed, dtype=torch.float64),
                "histories": torch.frombuffer(bytearray(buf.getvalue()), dtype=torch.uint8).clone()}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step = int(sd["step"])
        self.skipped_step = int(sd.get("skipped_step", 0))
        self.token = int(sd.get("token", 0))
        self.elapsed = float(sd.get("elapsed", 0.0))
        if "histories" in sd:
            hist = torch.load(io.BytesIO(sd["histories"].numpy().tobytes()), weights_only=False)
            self.global_avg_losses, self.global_max_losses, self.log_steps = hist["avg"], hist["max"], hist["steps"]


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _flatten(prefix: str, obj: Any, out: Dict[str, Any]) -> None:
    if isinstance(obj, dict):
        for k, v in obj.items():
            _flatten(f"{prefix}.{k}" if prefix else str(k), v, out)
    else:
        out[prefix] = obj


def _unflatten(flat: Dict[str, Any]) -> Dict[str, Any]:
    root: Dict[str, Any] = {}
    for key, v in flat.items():
        parts = key.split(".")
        cur = root
        for p in parts[:-1]:
            cur = cur.setdefault(p, {})
        cur[parts[-1]] = v
    return root


class CheckpointManager:
    def __init__(self, dump_folder: str, folder: str = "checkpoint", interval: int = 2048, keep_latest_k: int = 2,
                 save_backend: str = "dcp", model_weights_only: bool = False, export_dtype: str = "float32",
                 enable: bool = True, initial_load_path: Optional[str] = None,
                 exclude_from_loading: Optional[List[str]] = None, async_mode: str = "disabled"):
        if save_backend not in {"dcp", "rank0_model_only"}:
            raise ValueError("save_backend must be 'dcp' or 'rank0_model_only'")
        self.root = os.path.join(dump_folder, folder)
        self.interval = interval
        self.keep_latest_k = keep_latest_k
        self.save_backend = save_backend
        self.model_weights_only = model_weights_only
        self.export_dtype = getattr(torch, export_dtype)
        self.enable = enable
        self.initial_load_path = initial_load_path
        self.exclude_from_loading = set(exclude_from_loading or [])
        # "async" / "async_with_pinned_mem": the state is copied to host memory inside save() (collectively, so it
        # is a consistent snapshot of that step); rank 0 then writes and publishes it on a background thread while
        # training continues.  The next save, load or wait() joins the thread and re-raises its error, if any.
        if async_mode not in ("disabled", "async", "async_with_pinned_mem"):
            raise ValueError("async_mode must be 'disabled', 'async' or 'async_with_pinned_mem'")
        self.async_mode = async_mode
        self._writer = None
        self._writer_error: Optional[BaseException] = None

    # ------------------------------------------------------------------ discovery
    def steps(self) -> List[int]:
        if not os.path.isdir(self.root):
            return []
        out = []
        for name in os.listdir(self.root):
            m = _STEP_RE.match(name)
            if m and os.path.isdir(os.path.join(self.root, name)):
                out.append(int(m.group(1)))
        return sorted(out)

    def path(self, step: int) -> str:
        return os.path.join(self.root, f"step-{step}")

    def should_save(self, step: int, force: bool = False) -> bool:
        return self.enable and (force or (self.interval > 0 and step % self.interval == 0))

    def wait(self) -> None:
        """Block until a background write has been published; raise what it raised."""
        if self._writer is not None:
            self._writer.join()
            self._writer = None
        if self._writer_error is not None:
            err, self._writer_error = self._writer_error, None
            raise RuntimeError("asynchronous checkpoint write failed") from err

    # ------------------------------------------------------------------ save
    def save(self, step: int, model: torch.nn.Module, trainer=None, lr_scheduler=None, dataloader=None,
             train_state: Optional[TrainState] = None, force: bool = False) -> Optional[str]:
        if not self.should_save(step, force):
            return None
        self.wait()
        # live model state every time (the compute buffers are views that change in place)
        model_sd = {k: v.detach().to("cpu", self.export_dtype if v.is_floating_point() else v.dtype)
                    for k, v in model.state_dict().items()}
        opt_sd = None
        if trainer is not None and not self.model_weights_only and self.save_backend == "dcp":
            opt_sd = trainer.optimizer_state_dict()           # collective: gathers shards on every rank
            if trainer is not None:
                # parameters are stored from the fp32 masters, not from the bf16 compute copies
                for name, st in opt_sd["state"].items():
                    if name in model_sd and model_sd[name].is_floating_point():
                        model_sd[name] = st["master"].to(self.export_dtype).view(model_sd[name].shape)
        # every rank's data position goes into the checkpoint (collective; rank 0 writes all of them)
        loader_blobs: Optional[List[bytes]] = None
        if dataloader is not None and self.save_backend == "dcp":
            blob = io.BytesIO()
            torch.save(dataloader.state_dict(), blob)
            loader_blobs = [blob.getvalue()]
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                gathered: List[Any] = [None] * dist.get_world_size()
                dist.all_gather_object(gathered, loader_blobs[0])
                loader_blobs = gathered
        final = self.path(step)
        lr_sd = None if lr_scheduler is None else dict(lr_scheduler.state_dict())
        ts_sd = None if train_state is None else train_state.state_dict()

        def write() -> None:
            tmp = final + ".tmp"
            if os.path.exists(tmp):
                shutil.rmtree(tmp)
            os.makedirs(tmp, exist_ok=True)
            try:
                if self.save_backend == "rank0_model_only":
                    torch.save({"model": model_sd, "step": step}, os.path.join(tmp, "model.pt"))
                    with open(os.path.join(tmp, "metadata.json"), "w") as f:
                        json.dump({"step": step, "backend": "rank0_model_only", "time": time.time(),
                                   "num_tensors": len(model_sd)}, f)
                else:
                    states: Dict[str, Any] = {"model": model_sd}
                    if opt_sd is not None:
                        states["optimizer"] = {"step": torch.tensor(opt_sd["step"]),
                                               "skipped_steps": torch.tensor(opt_sd["skipped_steps"]),
                                               "state": opt_sd["state"]}
                    if lr_sd is not None:
                        states["lr_scheduler"] = {k: torch.tensor(v) if isinstance(v, (int, float)) else v
                                                  for k, v in lr_sd.items()}
                    if loader_blobs is not None:
                        states["dataloader"] = {f"rank_{r}": torch.frombuffer(bytearray(b), dtype=torch.uint8).clone()
                                                for r, b in enumerate(loader_blobs)}
                    if ts_sd is not None:
                        states["train_state"] = ts_sd
                    flat: Dict[str, Any] = {}
                    _flatten("", states, flat)
                    self._dcp_save(flat, tmp)
                if os.path.exists(final):
                    shutil.rmtree(final)
                os.replace(tmp, final)
            except BaseException:
                shutil.rmtree(tmp, ignore_errors=True)
                raise
            self._purge()

        if _rank() == 0:
            if self.async_mode == "disabled":
                write()
            else:
                import threading

                def guarded() -> None:
                    try:
                        write()
                    except BaseException as exc:      # surfaced by the next wait()
                        self._writer_error = exc
                self._writer = threading.Thread(target=guarded, name=f"checkpoint-step-{step}", daemon=False)
                self._writer.start()
        _barrier()
        return final

    @staticmethod
    def _dcp_save(flat: Dict[str, Any], path: str) -> None:
        import torch.distributed.checkpoint as dcp
        dcp.save(flat, storage_writer=dcp.FileSystemWriter(path, thread_count=1), no_dist=True)

    @staticmethod
    def _dcp_load(path: str) -> Dict[str, Any]:
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.default_planner import _EmptyStateDictLoadPlanner
        from torch.distributed.checkpoint.state_dict_loader import _load_state_dict
        sd: Dict[str, Any] = {}
        _load_state_dict(sd, storage_reader=dcp.FileSystemReader(path), planner=_EmptyStateDictLoadPlanner(),
                         no_dist=True)
        flat: Dict[str, Any] = {}
        _flatten("", sd, flat)
        return flat

    def _purge(self) -> None:
        if self.keep_latest_k <= 0:
            return
        steps = self.steps()
        for s in steps[:-self.keep_latest_k]:
            shutil.rmtree(self.path(s), ignore_errors=True)

    # ------------------------------------------------------------------ load
    def load(self, model: torch.nn.Module, trainer=None, lr_scheduler=None, dataloader=None,
             train_state: Optional[TrainState] = None, step: int = -1) -> Optional[int]:
        """Load ``step`` (newest readable when -1).  Missing keys are tolerated (partial load).
        Returns the step loaded or None when there is nothing to load."""
        self.wait()
        candidates: List[str] = []
        if step >= 0:
            candidates = [self.path(step)]
        else:
            candidates = [self.path(s) for s in reversed(self.steps())]
            if not candidates and self.initial_load_path:
                candidates = [self.initial_load_path]
        last_err: Optional[Exception] = None
        for path in candidates:
            try:
                loaded = self._load_path(path, model, trainer, lr_scheduler, dataloader, train_state)
                return loaded
            except (FileNotFoundError, MissingRankState):
                raise
            except Exception as exc:  # corrupt newest -> fall back to the previous one
                last_err = exc
                continue
        if last_err is not None:
            raise RuntimeError(f"no readable checkpoint under {self.root}") from last_err
        return None

    def _load_path(self, path, model, trainer, lr_scheduler, dataloader, train_state) -> int:
        if not os.path.isdir(path):
            raise FileNotFoundError(path)
        if os.path.exists(os.path.join(path, "model.pt")):
            blob = torch.load(os.path.join(path, "model.pt"), map_location="cpu", weights_only=False)
            self._load_model(model, blob["model"], trainer)
            return int(blob.get("step", 0))
        flat = self._dcp_load(path)
        states = _unflatten(flat)
        # model keys contain dots: recover them from the flat view
        model_sd = {k[len("model."):]: v for k, v in flat.items() if k.startswith("model.")}
        if "model" not in self.exclude_from_loading:
            self._load_model(model, model_sd, trainer)
        if trainer is not None and "optimizer" in states and "optimizer" not in self.exclude_from_loading:
            opt_flat = {k[len("optimizer.state."):]: v for k, v in flat.items() if k.startswith("optimizer.state.")}
            per_param: Dict[str, Dict[str, torch.Tensor]] = {}
            for k, v in opt_flat.items():
                name, key = k.rsplit(".", 1)
                per_param.setdefault(name, {})[key] = v
            trainer.load_optimizer_state_dict({"step": int(flat["optimizer.step"]),
                                               "skipped_steps": int(flat.get("optimizer.skipped_steps", 0)),
                                               "state": per_param})
        if lr_scheduler is not None and "lr_scheduler" in states and "lr_scheduler" not in self.exclude_from_loading:
            lr_scheduler.load_state_dict({k: (v.item() if torch.is_tensor(v) else v)
                                          for k, v in states["lr_scheduler"].items()})
        if dataloader is not None and "dataloader" in states and "dataloader" not in self.exclude_from_loading:
            key = f"rank_{_rank()}"
            if key not in states["dataloader"]:
                # resuming on more ranks than the checkpoint was written with: replaying data silently is worse
                # than stopping (exclude "dataloader" from loading to start the data over on purpose)
                raise MissingRankState(f"checkpoint {path} holds no data position for {key} "
                               f"(it has {sorted(states['dataloader'])})")
            dataloader.load_state_dict(torch.load(io.BytesIO(states["dataloader"][key].numpy().tobytes()),
                                                  weights_only=False))
        step = 0
        if train_state is not None and "train_state" in states:
            train_state.load_state_dict(states["train_state"])
            step = train_state.step
        elif "optimizer.step" in flat:
            step = int(flat["optimizer.step"])
        return step

    @staticmethod
    def _load_model(model, sd, trainer) -> None:
        own = model.state_dict()
        with torch.no_grad():
            for k, v in sd.items():
                if k in own and own[k].shape == v.shape:
                    own[k].copy_(v.to(own[k].dtype))
        if hasattr(getattr(model, "model", None), "_host_steps") and "model.memory_loss_free_steps" in sd:
            model.model._host_steps = int(sd["model.memory_loss_free_steps"])
        if trainer is not None:
            trainer.load_model_state()


def export_hf(model: torch.nn.Module, config, path: str, dtype: torch.dtype = torch.float32) -> None:
    """Write ``config.json`` + ``model.safetensors`` (falls back to ``pytorch_model.bin``)
    (uttt_llm/flame/utils/convert_dcp_to_hf.py:82-118)."""
    os.makedirs(path, exist_ok=True)
    config.save_pretrained(path)
    sd = {k: v.detach().to("cpu", dtype if v.is_floating_point() else v.dtype).contiguous()
          for k, v in model.state_dict().items()}
    try:
        from safetensors.torch import save_file
        save_file(sd, os.path.join(path, "model.safetensors"))
    except ImportError:
        torch.save(sd, os.path.join(path, "pytorch_model.bin"))
