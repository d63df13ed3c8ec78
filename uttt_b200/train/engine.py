"""Training engine: model + sharded optimizer + step function (the public training API).

``TrainEngine.train_step(batch)`` takes a batch in *host* memory (pinned when possible),
copies it to the device on a side stream, runs forward/backward over its micro-batches,
the fused gradient-reduce/clip/AdamW/redistribute step, and returns the loss as a device
tensor (call ``.item()`` / ``float()`` to read it back).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import LMConfig
from ..models import build_model
from ..parallel.fsdp import AdamWConfig, ShardedTrainer, lm_fsdp_units
from .lr import WarmupDecayLR


@dataclass
class EngineConfig:
    micro_batch_size: int = 1          # sequences per forward/backward
    lr: float = 1e-3
    eps: float = 1e-15
    beta1: float = 0.9
    beta2: float = 0.95
    weight_decay: float = 0.1
    max_norm: float = 1.0
    warmup_steps: int = 1024
    total_steps: int = 40960
    decay_type: str = "cosine"
    lr_min: float = 0.1
    skip_nan_inf: bool = True
    seed: int = 42
    activation_checkpoint: bool = True
    keep_activation_layers: tuple = ()     # layer indices that skip recomputation (needs spare device memory)
    activation_offload: bool = False       # saved tensors of the forward go to pinned host memory until backward
    data_parallel_replicate_degree: int = 1   # hybrid sharding: optimizer state sharded over world / R ranks, R replicas
    shard_parameters: bool = False         # ranks keep only their parameter shards between steps (library collectives)
    expert_capacity_factor: float = 2.0    # expert-parallel staging rows / balanced load (0 = size for the worst case)
    cuda_graph: bool = False               # replay forward + backward of a micro-batch as one CUDA graph
    cuda_graph_warmup: int = 2             # eager steps before the capture (lazy initialisation happens in them)


def init_distributed(backend: Optional[str] = None, timeout_seconds: Optional[float] = None,
                     trace_buf_size: Optional[int] = None) -> tuple[int, int, int]:
    """Join the torchrun rendezvous if there is one.  Returns (rank, world, local_rank).

    ``timeout_seconds`` bounds every collective until :func:`set_collective_timeout` tightens it after the first
    step (``comm.init_timeout_seconds`` / ``comm.train_timeout_seconds``, uttt_llm/flame/train.py:811-815);
    ``trace_buf_size`` sizes NCCL's flight recorder (``comm.trace_buf_size``)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        import datetime
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if trace_buf_size:
            os.environ.setdefault("TORCH_NCCL_TRACE_BUFFER_SIZE", str(int(trace_buf_size)))
        kwargs = {}
        if timeout_seconds:
            kwargs["timeout"] = datetime.timedelta(seconds=float(timeout_seconds))
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local), **kwargs)
        else:
            dist.init_process_group(backend, **kwargs)
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local


def set_collective_timeout(seconds: float) -> bool:
    """Tighten the time-out of the default process group (a rank that stops answering then fails the others'
    next collective after ``seconds`` instead of after the start-up allowance).  Returns False when the installed
    torch has no way to change it."""
    if not (dist.is_available() and dist.is_initialized()):
        return False
    import datetime
    try:
        from torch.distributed.distributed_c10d import _set_pg_timeout
        _set_pg_timeout(datetime.timedelta(seconds=float(seconds)), dist.group.WORLD)
        return True
    except Exception:
        return False


class _StepGraph:
    """A captured forward + backward: the graph, its static inputs and the output record it refreshes."""
    graph = None
    ids = labels = out = record = None
    launches = 0


class KernelStatusError(RuntimeError):
    """A bounded device-side wait gave up, or a staging buffer overflowed: results since then are not valid."""


class TrainEngine:
    def __init__(self, model_config: LMConfig, cfg: Optional[EngineConfig] = None,
                 device: Optional[torch.device] = None, model: Optional[nn.Module] = None):
        self.cfg = cfg or EngineConfig()
        self.model_config = model_config
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
        self.device = device
        torch.manual_seed(self.cfg.seed)   # same seed on every rank: identical initial weights
        if model is None:
            model = build_model(model_config)
        self.model = model.to(device)
        inner = getattr(self.model, "model", None)
        if inner is not None and hasattr(inner, "activation_checkpoint"):
            inner.activation_checkpoint = self.cfg.activation_checkpoint
            if hasattr(inner, "keep_activation_layers"):
                inner.keep_activation_layers = frozenset(int(i) for i in self.cfg.keep_activation_layers)
        self.expert_parallel = None
        ep_size = int(getattr(model_config, "memory_expert_parallel", 1) or 1)
        if ep_size > 1:
            import torch.distributed as dist
            from ..parallel.expert_parallel import ExpertParallel
            if not dist.is_initialized() or dist.get_world_size() % ep_size != 0:
                raise ValueError(f"memory_expert_parallel={ep_size} needs a job whose size is a multiple of it")
            world, rank = dist.get_world_size(), dist.get_rank()
            mine = None
            for start in range(0, world, ep_size):           # consecutive ranks share an NVLink domain
                grp = dist.new_group(list(range(start, start + ep_size)))
                if start <= rank < start + ep_size:
                    mine = grp
            self.expert_parallel = ExpertParallel(mine, device, model_config.memory_num_experts,
                                                  max_row_bytes=4 * model_config.fw_head_dim,
                                                  capacity_factor=float(self.cfg.expert_capacity_factor))
            inner.set_expert_parallel(self.expert_parallel)
        opt = AdamWConfig(lr=self.cfg.lr, beta1=self.cfg.beta1, beta2=self.cfg.beta2, eps=self.cfg.eps,
                          weight_decay=self.cfg.weight_decay, max_norm=self.cfg.max_norm,
                          skip_nan_inf=self.cfg.skip_nan_inf)
        shard_group, replicate_group = self._hybrid_groups(int(self.cfg.data_parallel_replicate_degree or 1))
        self.trainer = ShardedTrainer(self.model, lm_fsdp_units(self.model), opt, process_group=shard_group,
                                      replicate_group=replicate_group,
                                      shard_parameters=bool(self.cfg.shard_parameters))
        self.lr_sched = WarmupDecayLR(self.cfg.lr, self.cfg.total_steps, self.cfg.warmup_steps,
                                      self.cfg.decay_type, self.cfg.lr_min)
        self.copy_stream = torch.cuda.Stream(device) if device.type == "cuda" else None
        self.step = 0
        self.tokens_seen = 0
        self.last_stats: Dict[str, Any] = {}
        self._graphs: Dict[Any, "_StepGraph"] = {}
        self._graph_pool = None
        self.graph_error: Optional[str] = None     # why graph mode was given up, if it was

    @staticmethod
    def _hybrid_groups(replicas: int):
        """(shard group, replicate group) of this rank for hybrid sharding, or (None, None): consecutive ranks shard
        (they share an NVLink domain), ranks at the same position of every shard group replicate
        (uttt_llm/flame/models/parallelize_fla.py:632-648 builds the same two mesh dimensions)."""
        if replicas <= 1 or not (dist.is_available() and dist.is_initialized()):
            return None, None
        world, rank = dist.get_world_size(), dist.get_rank()
        if world % replicas != 0:
            raise ValueError(f"data_parallel_replicate_degree={replicas} does not divide the job size {world}")
        shard = world // replicas
        mine_s = mine_r = None
        for r in range(replicas):                       # every rank creates every group, in the same order
            g = dist.new_group(list(range(r * shard, (r + 1) * shard)))
            if r * shard <= rank < (r + 1) * shard:
                mine_s = g
        for j in range(shard):
            g = dist.new_group([r * shard + j for r in range(replicas)])
            if rank % shard == j:
                mine_r = g
        return mine_s, mine_r

    # ------------------------------------------------------------------ data movement
    def to_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        if self.copy_stream is None:
            return {k: v.to(self.device) for k, v in batch.items()}
        with torch.cuda.stream(self.copy_stream):
            out = {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}
        torch.cuda.current_stream(self.device).wait_stream(self.copy_stream)
        return out

    # ------------------------------------------------------------------ one optimizer step
    def train_step(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        """batch: {'input_ids': [B, S], 'labels': [B, S]} (host or device).  Returns the mean loss (device)."""
        self.model.train()
        ids_all = batch["input_ids"]
        if ids_all.device != self.device:
            batch = self.to_device(batch)
            ids_all = batch["input_ids"]
        labels_all = batch.get("labels", ids_all)
        bsz = ids_all.shape[0]
        mb = min(self.cfg.micro_batch_size, bsz)
        n_micro = (bsz + mb - 1) // mb
        total = torch.zeros((), device=self.device, dtype=torch.float32)
        self.trainer.gather_params()                   # no-op unless the parameters are sharded between steps
        for i in range(n_micro):
            ids, labels = ids_all[i * mb:(i + 1) * mb], labels_all[i * mb:(i + 1) * mb]
            out = self._replay_forward_backward(ids, labels, n_micro) if self._graph_ready() else None
            if out is None:
                with self._offload():
                    out = self.model(input_ids=ids, labels=labels)
                (out.loss / n_micro).backward()
            total += out.loss.detach().float() / n_micro
            if n_micro > 1:
                self.trainer.accumulate_micro_batch()
            if i == n_micro - 1:
                self.trainer.release_params()          # parameter-sharded mode: the full buffers go before the optimizer runs
            self.last_stats = {"ce": out.ce_loss, "lb": out.lb_loss}
            moe = (getattr(out, "moe_stats", None) or {}).get("moe")
            if moe:
                self.last_stats["moe"] = moe
        lr = self.lr_sched.lr()
        stats = self.trainer.step(lr=lr)
        self.lr_sched.step()
        self.step += 1
        self.tokens_seen += ids_all.numel()
        self.last_stats.update(stats)
        self.last_stats["lr"] = lr
        return total

    # ------------------------------------------------------------------ forward + backward as one CUDA graph
    def _graph_ready(self) -> bool:
        return (self.cfg.cuda_graph and self.graph_error is None and self.device.type == "cuda"
                and self.step >= self.cfg.cuda_graph_warmup and self.expert_parallel is None
                and not self.cfg.activation_offload
                # a graph replays fixed addresses: not with parameter buffers that are dropped and brought back
                and not self.trainer.shard_parameters)

    def _host_branches(self):
        """What the model's next training forward decides on the host (not on the device): a captured graph is
        only valid for the decisions it was captured with."""
        inner = getattr(self.model, "model", self.model)
        fn = getattr(inner, "host_branch_key", None)
        return fn() if fn is not None else ()

    def _replay_forward_backward(self, ids: torch.Tensor, labels: torch.Tensor, n_micro: int):
        """Forward + backward of one micro-batch from a captured graph (captured on first use for this input shape
        and these host-side decisions).  The step is launch-bound otherwise: tens of thousands of small launches per
        step keep the host busier than the device.  Returns None when this step has to run eagerly."""
        branches = self._host_branches()
        if branches is None:                       # e.g. a statistics step: host-side reads in the forward
            return None
        key = (tuple(ids.shape), ids.dtype, n_micro, branches)
        sg = self._graphs.get(key)
        if sg is None:
            try:
                sg = self._capture(ids, labels, n_micro)
            except Exception as exc:               # capture refused an operation: stay eager from here on
                self.graph_error = f"{type(exc).__name__}: {exc}"
                return None                        # (a failed capture executed nothing: gradients are untouched)
            self._graphs[key] = sg
        sg.ids.copy_(ids)
        sg.labels.copy_(labels)
        sg.graph.replay()
        from ..ops import functional as F
        F._count(sg.launches)
        inner = getattr(self.model, "model", self.model)
        done = getattr(inner, "host_step_replayed", None)
        if done is not None:
            done(sg.record)
        return sg.out

    def _capture(self, ids: torch.Tensor, labels: torch.Tensor, n_micro: int) -> "_StepGraph":
        from ..ops import functional as F
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()                   # the eager steps' cached blocks go back before the graph's pool grows
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        sg = _StepGraph()
        sg.ids, sg.labels = ids.clone(), labels.clone()
        sg.graph = torch.cuda.CUDAGraph()
        inner = getattr(self.model, "model", self.model)
        host = inner.host_state() if hasattr(inner, "host_state") else None
        before = F.launch_count()
        try:
            with torch.cuda.graph(sg.graph, pool=self._graph_pool):
                out = self.model(input_ids=sg.ids, labels=sg.labels)
                (out.loss / n_micro).backward()
        finally:
            if host is not None:                   # the capture ran the host side of a step, not the device side
                inner.load_host_state(host)
        sg.launches = F.launch_count() - before
        sg.record = inner.pop_capture_record() if hasattr(inner, "pop_capture_record") else None
        out.hidden_states = None                   # nothing outside needs the hidden states of a replayed step
        sg.out = out
        return sg

    def release_graphs(self) -> None:
        """Drop the captured graphs and their memory pool (before the process group goes away, or to return to
        eager steps with the memory they hold)."""
        self._graphs.clear()
        self._graph_pool = None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            torch.cuda.empty_cache()

    def _offload(self):
        from ..utils.activation_offload import offload_activations
        return offload_activations(enabled=self.cfg.activation_offload and self.device.type == "cuda")

    def kernel_status(self) -> int:
        """The device status word of the tensor-core / expert-parallel kernels (0 = healthy).  Reading it
        synchronises with the device: call it at log and checkpoint steps, not every step."""
        if self.device.type != "cuda":
            return 0
        from ..ops._ext import load
        ext = load()
        if ext is None or not hasattr(ext, "gemm_status"):
            return 0
        return int(ext.gemm_status(torch.zeros(1, device=self.device))[0].item())

    def check_kernel_status(self) -> None:
        """Raise when a kernel reported a failed bounded wait or an overflow.  After such a report every later
        tensor-core kernel returns at once and leaves its outputs stale, so training must not go on (and no
        checkpoint may be written) on top of it."""
        code = self.kernel_status()
        if code != 0:
            raise KernelStatusError(
                f"device status word = {code} at step {self.step}: a bounded wait timed out (codes 1-59), an "
                f"expert-parallel staging buffer overflowed (61) or an index was out of range (7x); "
                f"restart from the last checkpoint")

    @torch.no_grad()
    def eval_loss(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        self.model.eval()
        batch = self.to_device(batch) if batch["input_ids"].device != self.device else batch
        out = self.model(input_ids=batch["input_ids"], labels=batch.get("labels", batch["input_ids"]))
        return out.loss
