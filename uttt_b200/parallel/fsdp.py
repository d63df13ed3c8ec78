"""Flat-buffer fully-sharded data parallelism with the optimizer fused into the gradient path.

What the reference does with FSDP2 (uttt_llm/flame/models/parallelize_fla.py:470-571: one
unit per block plus a root unit, bf16 parameters, fp32 gradient reduction, parameters kept
unsharded for the whole step) is done here with explicit flat buffers:

* every unit owns one contiguous *compute* buffer (bf16 on GPU) that all its parameters view,
  one contiguous low-precision gradient buffer that all ``param.grad`` view, and fp32
  master / exp_avg / exp_avg_sq *shards* (1/world of the unit each);
* ``step()`` = reduce-scatter of the gradient buffer into the local fp32 shard, global-norm
  clip, AdamW on the shard, and redistribution of the updated bf16 shard into every rank's
  compute buffer.  On CUDA with symmetric memory this is two kernels per unit that read peers'
  gradient buffers and write peers' compute buffers directly over NVLink
  (:mod:`uttt_b200.parallel.symm`); elsewhere it is ``torch.distributed`` collectives.

The engine is independent of the model: it only needs a list of (name, parameter) units.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import reference as ref
from ..ops._ext import cuda_ext

_ALIGN = 256  # elements; keeps every shard 512-byte aligned in bf16 and 1 KiB aligned in fp32


def _dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    weight_decay: bool


class FlatUnit:
    """One sharding unit: a flat compute buffer, a flat gradient buffer and fp32 shards."""

    def __init__(self, name: str, named_params: Sequence[Tuple[str, nn.Parameter]], world: int, rank: int,
                 compute_dtype: torch.dtype, no_decay: Callable[[str, nn.Parameter], bool], allocator=None):
        self.name = name
        self.world, self.rank = world, rank
        device = named_params[0][1].device
        self.slots: List[ParamSlot] = []
        # decayed parameters first, then non-decayed: each shard sees at most one boundary
        ordered = sorted(named_params, key=lambda np_: no_decay(np_[0], np_[1]))
        off = 0
        for pname, p in ordered:
            self.slots.append(ParamSlot(pname, p, off, p.numel(), not no_decay(pname, p)))
            off += (p.numel() + 7) // 8 * 8
        self.decay_end = next((s.offset for s in self.slots if not s.weight_decay), off)
        chunk = _ALIGN * world
        self.numel = (off + chunk - 1) // chunk * chunk
        self.shard_numel = self.numel // world
        alloc = allocator or (lambda n, dtype: torch.zeros(n, dtype=dtype, device=device))
        self.compute = alloc(self.numel, compute_dtype)
        self.grad = alloc(self.numel, compute_dtype)
        self.compute.zero_()
        self.grad.zero_()
        lo = rank * self.shard_numel
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        with torch.no_grad():
            full = torch.zeros(self.numel, dtype=torch.float32, device=device)
            for s in self.slots:
                full[s.offset:s.offset + s.numel] = s.param.detach().float().reshape(-1)
            self.master.copy_(full[lo:lo + self.shard_numel])
            self.compute.copy_(full)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_accum: Optional[torch.Tensor] = None  # fp32 full-size, only with >1 micro-batch
        for s in self.slots:
            s.param.data = self.compute[s.offset:s.offset + s.numel].view(s.param.shape)
            s.param.grad = self.grad[s.offset:s.offset + s.numel].view(s.param.shape)

    @property
    def shard_range(self) -> Tuple[int, int]:
        lo = self.rank * self.shard_numel
        return lo, lo + self.shard_numel

    def rebind_grads(self) -> None:
        for s in self.slots:
            g = self.grad[s.offset:s.offset + s.numel].view(s.param.shape)
            if s.param.grad is None or s.param.grad.data_ptr() != g.data_ptr():
                if s.param.grad is not None:
                    g.add_(s.param.grad.to(g.dtype))
                s.param.grad = g


def default_no_decay(name: str, p: nn.Parameter) -> bool:
    """Parameters excluded from weight decay by name suffix (uttt_llm/flame/components/optimizer.py:20-60)."""
    leaf = name.rsplit(".", 1)[-1]
    return leaf.startswith("prev_chunk_alpha") or name.endswith((".A_log", ".dt_bias", ".D"))


@dataclass
class AdamWConfig:
    lr: float = 8e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    max_norm: float = 1.0
    skip_nan_inf: bool = True


class ShardedTrainer:
    """Owns the flat units of a model and runs the fused gradient-reduce / clip / AdamW / gather step."""

    def __init__(self, model: nn.Module, unit_modules: Optional[Sequence[Tuple[str, nn.Module]]] = None,
                 opt: Optional[AdamWConfig] = None, compute_dtype: Optional[torch.dtype] = None,
                 no_decay: Callable[[str, nn.Parameter], bool] = default_no_decay, process_group=None,
                 use_symmetric_memory: Optional[bool] = None, replicate_group=None, shard_parameters: bool = False):
        """``process_group``: the ranks that shard the optimizer state (default: all).  ``replicate_group``: the ranks
        that hold the same shard in other shard groups (hybrid sharding: gradients are reduce-scattered inside a shard
        group and all-reduced across the replicas of each shard; ``training.data_parallel_replicate_degree``).
        ``shard_parameters``: between steps a rank keeps only its shard of the low-precision parameters; the full
        buffers are gathered before the model runs and dropped after backward (``release_params``).  This mode uses
        library collectives (the peer-memory optimizer kernels write every rank's full buffer, which it does not have)."""
        self.model = model
        self.opt = opt or AdamWConfig()
        self.group = process_group
        self.world = dist.get_world_size(process_group) if _dist_ready() else 1
        self.rank = dist.get_rank(process_group) if _dist_ready() else 0
        self.replicate_group = replicate_group
        self.replicas = dist.get_world_size(replicate_group) if (_dist_ready() and replicate_group is not None) else 1
        first = next(model.parameters())
        self.device = first.device
        if compute_dtype is None:
            compute_dtype = torch.bfloat16 if first.is_cuda else torch.float32
        self.compute_dtype = compute_dtype
        self.step_count = 0
        self.skipped_steps = 0
        self.micro_batches = 0
        self.symm = None
        self.shard_parameters = bool(shard_parameters) and self.world > 1
        self.params_released = False
        if self.shard_parameters:
            use_symmetric_memory = False
        if use_symmetric_memory is None:
            use_symmetric_memory = first.is_cuda and self.world > 1
        # --- partition parameters into units: one per listed module, the remainder is the root unit
        seen = set()
        units: List[Tuple[str, List[Tuple[str, nn.Parameter]]]] = []
        prefix_of = {}
        for uname, mod in (unit_modules or []):
            plist = []
            for pn, p in mod.named_parameters():
                if id(p) in seen:
                    continue
                seen.add(id(p))
                plist.append((f"{uname}.{pn}", p))
            if plist:
                units.append((uname, plist))
        root = [(pn, p) for pn, p in model.named_parameters() if id(p) not in seen and not seen.add(id(p))]
        if root:
            units.append(("root", root))
        if use_symmetric_memory:
            try:
                from .symm import SymmetricHeap
                item = torch.empty((), dtype=compute_dtype).element_size()
                chunk = _ALIGN * self.world
                total = 0
                for _, pl in units:
                    n = sum((p.numel() + 7) // 8 * 8 for _, p in pl)
                    n = (n + chunk - 1) // chunk * chunk
                    # compute + low-precision grad + (optional) fp32 accumulation buffer, 1 KiB aligned each
                    total += n * item * 2 + n * 4 + 3 * 1024
                self.symm = SymmetricHeap(self.device, self.group, capacity_bytes=total + (1 << 20))
            except Exception as exc:  # pragma: no cover - depends on the box
                import warnings
                warnings.warn(f"symmetric memory unavailable ({exc}); gradient path falls back to NCCL collectives")
                self.symm = None
        alloc = self.symm.alloc if self.symm is not None else None
        self.units = [FlatUnit(n, pl, self.world, self.rank, compute_dtype, no_decay, alloc) for n, pl in units]
        # tied / aliased tensors (e.g. tied embeddings) keep working: every alias views the same slot
        for buf_name, buf in model.named_buffers():
            if buf.is_floating_point() and buf.dtype != torch.float32 and "loss_free" in buf_name:
                buf.data = buf.data.float()
        self._norm_buf = torch.zeros(2, dtype=torch.float32, device=self.device)
        if self.shard_parameters:
            for u in self.units:
                lo, hi = u.shard_range
                u.compute_shard = u.compute[lo:hi].clone()
            # whoever runs the model or asks for its state finds the parameters gathered
            model.register_forward_pre_hook(lambda *_: self.gather_params())
            model.register_state_dict_pre_hook(lambda *_: self.gather_params())
        if self.symm is not None:
            self.symm.finalize()
        if self.device.type == "cuda":
            # the .grad tensors are persistent views of the flat buffers: dense projections may add their weight
            # gradients into them inside the GEMM
            from ..ops import set_fused_weight_grad
            set_fused_weight_grad(True)

    # ------------------------------------------------------------------ parameter sharding
    def release_params(self) -> None:
        """Drop the full low-precision parameter buffers (each rank keeps its shard).  Call after backward."""
        if not self.shard_parameters or self.params_released:
            return
        for u in self.units:
            lo, hi = u.shard_range
            u.compute_shard.copy_(u.compute[lo:hi])
            u.compute.untyped_storage().resize_(0)
        self.params_released = True

    def gather_params(self) -> None:
        """Bring the full parameter buffers back from the ranks' shards (no-op while they are present)."""
        if not self.shard_parameters or not self.params_released:
            return
        for u in self.units:
            u.compute.untyped_storage().resize_(u.numel * u.compute.element_size())
            dist.all_gather_into_tensor(u.compute, u.compute_shard, group=self.group)
        self.params_released = False

    def _param_shard(self, u: "FlatUnit") -> torch.Tensor:
        """Where the optimizer writes this rank's new low-precision parameters."""
        if self.shard_parameters and self.params_released:
            return u.compute_shard
        lo, hi = u.shard_range
        return u.compute[lo:hi]

    # ------------------------------------------------------------------ bookkeeping
    def num_parameters(self) -> int:
        return sum(s.numel for u in self.units for s in u.slots)

    def zero_grad(self) -> None:
        for u in self.units:
            u.grad.zero_()
            u.rebind_grads()
            if u.grad_accum is not None:
                u.grad_accum.zero_()
        self.micro_batches = 0

    def accumulate_micro_batch(self) -> None:
        """Fold the low-precision gradient buffer into fp32 accumulators between micro-batches.

        Only needed when a step has more than one micro-batch; a single micro-batch is reduced
        straight from the low-precision buffer with fp32 accumulation inside the reduce kernel.
        """
        for u in self.units:
            u.rebind_grads()
            if u.grad_accum is None:
                u.grad_accum = (self.symm.alloc(u.numel, torch.float32).zero_() if self.symm is not None
                                else torch.zeros(u.numel, dtype=torch.float32, device=self.device))
            u.grad_accum.add_(u.grad)
            u.grad.zero_()
        self.micro_batches += 1

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, lr: Optional[float] = None, grad_divisor: float = 1.0,
             skip_above: Optional[float] = None) -> Dict[str, torch.Tensor]:
        """Reduce gradients (mean over ranks, divided by ``grad_divisor``), clip, AdamW, redistribute.

        Returns {'grad_norm': tensor, 'skipped': tensor(bool)} without a host sync.
        """
        opt = self.opt
        lr = opt.lr if lr is None else lr
        self.step_count += 1
        scale = 1.0 / (self.world * self.replicas * grad_divisor)
        hybrid = self.replicas > 1
        shards: List[torch.Tensor] = []
        sq = torch.zeros((), dtype=torch.float32, device=self.device)
        fused = self.symm is not None
        if fused:
            self.symm.barrier()          # every rank's backward has finished writing its gradient buffer
        ext = cuda_ext(self.units[0].master) if self.units else None
        native = ext is not None and hasattr(ext, "adamw_flat")
        gmuls: List[float] = []
        sq1 = sq.view(1)
        for u in self.units:
            u.rebind_grads()
            src = u.grad_accum if u.grad_accum is not None else u.grad
            gmul = 1.0
            if fused:
                g = self.symm.reduce_scatter_sumsq(u, src, scale, torch.zeros_like(sq1) if hybrid else sq1)
            elif self.world > 1:
                g = torch.empty(u.shard_numel, dtype=torch.float32, device=self.device)
                dist.reduce_scatter_tensor(g, src.float(), group=self.group)
                g.mul_(scale)
                if not hybrid:
                    sq += g.pow(2).sum()
            elif hybrid:
                g = src.float() * scale
            elif native:
                # single rank: the optimizer kernel reads the gradient buffer in place
                g, gmul = src, scale
                ext.sumsq_accum(src, float(scale), sq1)
            else:
                g = src.float() * scale if scale != 1.0 or src.dtype != torch.float32 else src
                sq += g.pow(2).sum()
            if hybrid:
                # the same shard of the other shard groups: sum across the replicas, then its share of the norm
                dist.all_reduce(g, group=self.replicate_group)
                sq += g.float().pow(2).sum()
            shards.append(g)
            gmuls.append(gmul)
        if self.world > 1:
            dist.all_reduce(sq, group=self.group)
        grad_norm = sq.sqrt()
        finite = torch.isfinite(grad_norm)
        if skip_above is not None:
            # caller's outlier rule: a step whose gradient norm exceeds the threshold is skipped like a NaN step
            finite = finite & (grad_norm <= skip_above)
        clip = torch.ones_like(grad_norm)
        if opt.max_norm and opt.max_norm > 0:
            clip = (opt.max_norm / (grad_norm + 1e-6)).clamp(max=1.0)
        # a non-finite norm turns the update into a no-op (skip_nan_inf) without branching on the host
        gscale = torch.where(finite, clip, torch.zeros_like(clip)) if opt.skip_nan_inf else clip
        apply = finite.float() if opt.skip_nan_inf else torch.ones_like(clip)
        gscale1, apply1 = gscale.reshape(1).float(), apply.reshape(1).float()
        for u, g, gmul in zip(self.units, shards, gmuls):
            self._adamw_unit(u, g, lr, gscale1, apply1, gmul)
        if fused:
            self.symm.barrier()          # all peers' compute buffers now hold the new parameters
        for u in self.units:
            u.grad.zero_()
            if u.grad_accum is not None:
                u.grad_accum.zero_()
        self.micro_batches = 0
        return {"grad_norm": grad_norm, "skipped": ~finite}

    def _adamw_unit(self, u: FlatUnit, g: torch.Tensor, lr: float, gscale: torch.Tensor, apply: torch.Tensor,
                    gmul: float = 1.0):
        opt = self.opt
        lo, hi = u.shard_range
        decay_hi = min(max(u.decay_end - lo, 0), u.shard_numel)   # elements [0, decay_hi) of the shard decay
        ext = cuda_ext(u.master)
        if ext is not None and hasattr(ext, "adamw_flat"):
            if self.symm is not None:
                self.symm.adamw_scatter(u, g, lr, opt, self.step_count, gscale, apply, decay_hi)
                return
            ext.adamw_flat(u.master, g, u.exp_avg, u.exp_avg_sq, self._param_shard(u), float(lr), opt.beta1, opt.beta2,
                           opt.eps, opt.weight_decay, int(self.step_count), gscale, apply, float(gmul),
                           int(decay_hi))
        else:
            self._adamw_torch(u, g, lr, gscale, apply, decay_hi)
        # without the peer-memory kernels the other ranks' shards arrive through a library all-gather (unless the
        # full buffers are released: then they are gathered before the next forward)
        if self.world > 1 and not (self.shard_parameters and self.params_released):
            dist.all_gather_into_tensor(u.compute, u.compute[lo:hi].clone(), group=self.group)

    def _adamw_torch(self, u, g, lr, gscale, apply, decay_hi):
        opt = self.opt
        lo, hi = u.shard_range
        gf = g.float() * gscale
        b1, b2 = opt.beta1, opt.beta2
        step = self.step_count
        m_new = u.exp_avg * b1 + gf * (1 - b1)
        v_new = u.exp_avg_sq * b2 + gf * gf * (1 - b2)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        decay = torch.ones_like(u.master)
        decay[:decay_hi] = 1 - lr * opt.weight_decay
        p_new = u.master * decay - (lr / bc1) * m_new / (v_new.sqrt() / math.sqrt(bc2) + opt.eps)
        keep = apply > 0
        u.exp_avg.copy_(torch.where(keep, m_new, u.exp_avg))
        u.exp_avg_sq.copy_(torch.where(keep, v_new, u.exp_avg_sq))
        u.master.copy_(torch.where(keep, p_new, u.master))
        self._param_shard(u).copy_(u.master)

    # ------------------------------------------------------------------ state dict (full, rank-agnostic)
    def _gather_shards(self, shard: torch.Tensor, u: FlatUnit) -> torch.Tensor:
        if self.world == 1:
            return shard
        full = torch.empty(u.numel, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def optimizer_state_dict(self) -> Dict[str, Dict[str, torch.Tensor]]:
        """Per-parameter fp32 master / moments keyed by parameter name (identical on every rank)."""
        out: Dict[str, Dict[str, torch.Tensor]] = {}
        for u in self.units:
            fulls = {k: self._gather_shards(getattr(u, k), u) for k in ("master", "exp_avg", "exp_avg_sq")}
            for s in u.slots:
                out[s.name] = {k: v[s.offset:s.offset + s.numel].view(s.param.shape).clone().cpu()
                               for k, v in fulls.items()}
        return {"step": self.step_count, "skipped_steps": self.skipped_steps, "state": out}

    def load_optimizer_state_dict(self, sd: Dict) -> None:
        self.step_count = int(sd.get("step", 0))
        self.skipped_steps = int(sd.get("skipped_steps", 0))
        state = sd["state"]
        for u in self.units:
            lo, hi = u.shard_range
            for key in ("master", "exp_avg", "exp_avg_sq"):
                full = torch.zeros(u.numel, dtype=torch.float32, device=self.device)
                present = False
                for s in u.slots:
                    if s.name in state and key in state[s.name]:
                        full[s.offset:s.offset + s.numel] = state[s.name][key].reshape(-1).to(self.device)
                        present = True
                    elif key == "master":
                        full[s.offset:s.offset + s.numel] = s.param.detach().float().reshape(-1)
                if present or key == "master":
                    getattr(u, key).copy_(full[lo:hi])
            self.sync_compute_from_master(u)

    @torch.no_grad()
    def sync_compute_from_master(self, u: Optional[FlatUnit] = None) -> None:
        for unit in ([u] if u is not None else self.units):
            full = self._gather_shards(unit.master, unit)
            unit.compute.copy_(full)

    @torch.no_grad()
    def load_model_state(self) -> None:
        """Re-read parameter values (e.g. after ``load_state_dict``) into the fp32 master shards."""
        for u in self.units:
            lo, hi = u.shard_range
            full = u.compute.float()
            u.master.copy_(full[lo:hi])


def lm_fsdp_units(model: nn.Module) -> List[Tuple[str, nn.Module]]:
    """Per-block units for a causal LM (the remainder - embeddings, head, pool, routers - is the root unit)."""
    layers = getattr(getattr(model, "model", model), "layers", None)
    prefix = "model.layers" if hasattr(model, "model") else "layers"
    return [] if layers is None else [(f"{prefix}.{i}", blk) for i, blk in enumerate(layers)]
