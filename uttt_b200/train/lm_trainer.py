"""Language-model training entry point:  ``torchrun -m uttt_b200.train.lm_trainer --job.config_file job.toml
--model.config model.json [--section.key value ...]``.

The loop follows the reference trainer (uttt_llm/flame/train.py:156-822): distributed init, data source,
model build from the architecture JSON, sharding, optimizer + schedule, checkpoint resume, gradient
accumulation, clipping with NaN/Inf step skipping, periodic metrics (loss average / max over ranks,
tokens/s, MFU, memory), checkpointing, optional torch profiler traces.  Differences: the global-batch guard
(``training.expected_global_batch_size``) is checked before anything is allocated; the loss-free balancing
interval is multiplied by the accumulation factor as in the reference (:282-292); device timing uses CUDA
events; the gradient path is the fused peer-memory reduce/AdamW/all-gather step.
"""
from __future__ import annotations

import gc
import json
import os
import sys
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..config import load_config
from ..config.job_config import JobConfig
from ..utils.flops import get_nparams_and_flops, peak_flops
from .checkpoint import CheckpointManager, TrainState
from .data import build_dataloader
from .engine import EngineConfig, TrainEngine, init_distributed, set_collective_timeout


def check_global_batch(job: JobConfig, world: int) -> int:
    got = job.training.batch_size * world * job.training.gradient_accumulation_steps
    want = job.training.expected_global_batch_size
    if want is not None and int(want) != got:
        raise ValueError(f"training.batch_size ({job.training.batch_size}) x data-parallel ranks ({world}) x "
                         f"gradient_accumulation_steps ({job.training.gradient_accumulation_steps}) = {got}, "
                         f"but training.expected_global_batch_size = {want}")
    return got


class Metrics:
    """Loss history + throughput bookkeeping; prints, and writes TensorBoard / JSONL when enabled."""

    def __init__(self, job: JobConfig, rank: int, flops_per_token: float, n_gpus: int):
        self.rank, self.job = rank, job
        self.flops_per_token, self.n_gpus = flops_per_token, n_gpus
        self.t_last, self.tokens_since = time.perf_counter(), 0
        self.path = os.path.join(job.job.dump_folder, "metrics.jsonl")
        self.tb = None
        self.wandb = None
        if rank == 0 and job.metrics.enable_wandb and os.environ.get("DISABLE_WANDB", "0").lower() in ("0", "", "false"):
            try:
                import wandb
            except ImportError as exc:
                raise ImportError("metrics.enable_wandb is set but the wandb package is not installed; install it "
                                  "or set DISABLE_WANDB=1 (metrics still go to stdout, metrics.jsonl and "
                                  "TensorBoard)") from exc
            self.wandb = wandb.init(project=os.environ.get("WANDB_PROJECT", "uttt_b200"),
                                    name=os.environ.get("WANDB_NAME"), dir=job.job.dump_folder,
                                    config=job.to_dict(), resume="allow")
        if rank == 0:
            os.makedirs(job.job.dump_folder, exist_ok=True)
            if job.metrics.enable_tensorboard:
                try:
                    from torch.utils.tensorboard import SummaryWriter
                    self.tb = SummaryWriter(os.path.join(job.job.dump_folder, job.metrics.save_tb_folder))
                except Exception:
                    self.tb = None

    def log(self, step: int, loss: torch.Tensor, stats: Dict[str, Any], tokens: int, state: TrainState) -> None:
        self.tokens_since += tokens
        if step % self.job.metrics.log_freq != 0 and step != 1:
            return
        avg, mx = loss.detach().float().clone(), loss.detach().float().clone()
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(avg, op=dist.ReduceOp.AVG)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        now = time.perf_counter()
        dt = max(now - self.t_last, 1e-9)
        tps = self.tokens_since / dt                       # per rank
        mfu = 100.0 * self.flops_per_token * tps / peak_flops()
        self.t_last, self.tokens_since = now, 0
        state.global_avg_losses.append(float(avg))
        state.global_max_losses.append(float(mx))
        state.log_steps.append(step)
        if self.rank == 0:
            mem = torch.cuda.max_memory_reserved() / 2 ** 30 if torch.cuda.is_available() else 0.0
            rec = {"step": step, "loss": float(avg), "loss_max": float(mx), "tps_per_gpu": tps, "mfu": mfu,
                   "memory_gib": mem, "lr": stats.get("lr"), "grad_norm": float(stats["grad_norm"]),
                   "skipped_step": state.skipped_step}
            for k in ("ce", "lb"):
                if stats.get(k) is not None:
                    rec[f"loss/{k}"] = float(stats[k])
            for k, v in (stats.get("moe") or {}).items():          # pool statistics, on their interval
                rec[f"moe/{k}"] = float(v)
            print(f"step {step:6d}  loss {rec['loss']:.4f}  grad_norm {rec['grad_norm']:.3f}  lr {rec['lr']:.2e}  "
                  f"tps/gpu {tps:,.0f}  mfu {mfu:.1f}%  mem {mem:.1f} GiB", flush=True)
            with open(self.path, "a") as fh:
                fh.write(json.dumps(rec) + "\n")
            if self.tb is not None:
                for k, v in rec.items():
                    if isinstance(v, (int, float)) and k != "step":
                        self.tb.add_scalar(k, v, step)
            if self.wandb is not None:
                self.wandb.log({k: v for k, v in rec.items() if isinstance(v, (int, float))}, step=step)


def param_check(model: torch.nn.Module) -> List[str]:
    """One line per parameter with its shape, mean and standard deviation (the reference prints the same table
    at start-up, uttt_llm/flame/train.py:394-420): a wrong initialisation or a failed load shows up before step 1."""
    lines = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            f = p.detach().float()
            std = float(f.std()) if f.numel() > 1 else 0.0
            lines.append(f"[param-check] {name} shape={tuple(p.shape)} mean={float(f.mean()):+.6e} std={std:.6e}")
    return lines


def estimate_memory(model_cfg, job: JobConfig, world: int) -> Dict[str, float]:
    """Analytic per-GPU memory estimate in GiB (``memory_estimation.enabled``): parameters and optimizer state from
    a meta-device build, fast-weight state and recompute checkpoints from the shapes of the chunk recurrence."""
    from ..models import build_model
    with torch.device("meta"):
        n = sum(p.numel() for p in build_model(model_cfg).parameters())
    b, s = job.training.batch_size, job.training.seq_len
    d, layers = model_cfg.hidden_size, model_cfg.num_hidden_layers
    chunk = getattr(model_cfg, "chunk_size", s) or s
    gib = 2.0 ** 30
    out = {"params_bf16": 2 * n / gib, "grads_bf16": 2 * n / gib, "optimizer_fp32_shard": 12 * n / max(world, 1) / gib}
    if getattr(model_cfg, "use_memory_block", False) and hasattr(model_cfg, "memory_num_experts"):
        e, hd, inter = model_cfg.memory_num_experts, model_cfg.fw_head_dim, model_cfg.fw_inter_dim
        per_seq = 3 * e * hd * inter * (4 + 4 + 2)                        # master + momentum + compute copy
        out["pool_state_per_version"] = b * per_seq / gib
        out["pool_versions_kept_for_backward"] = out["pool_state_per_version"] * (s // chunk)
    out["chunk_checkpoints"] = b * s * d * 2 * layers / gib               # one block input per (chunk, layer)
    out["recompute_working_set"] = b * chunk * d * 2 * 40 / gib           # activations of one (chunk, layer) region
    out["logits_chunk"] = 8192 * model_cfg.vocab_size * 2 * 2 / gib
    out["total"] = sum(out.values())
    return out


def main(job: Optional[JobConfig] = None) -> TrainState:
    job = job or JobConfig().parse_args()
    rank, world, local = init_distributed(timeout_seconds=job.comm.init_timeout_seconds,
                                          trace_buf_size=job.comm.trace_buf_size)
    check_global_batch(job, world)
    if job.job.print_args and rank == 0:
        print(json.dumps(job.to_dict(), indent=1, default=str))
    if job.training.deterministic:
        # same seed, same reduction order: bit-identical reruns (the kernels of this framework use fixed
        # reduction orders except the embedding-gradient scatter, which uses fp32 reductions in memory)
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic, torch.backends.cudnn.benchmark = True, False
    model_cfg = load_config(job.model.config)
    if job.experimental.expert_parallel_degree > 1:
        model_cfg = model_cfg.replace(memory_expert_parallel=int(job.experimental.expert_parallel_degree))
    if job.memory_estimation.enabled:
        est = estimate_memory(model_cfg, job, world)
        if rank == 0:
            print("[memory-estimate] " + " ".join(f"{k}={v:.2f}GiB" for k, v in est.items()), flush=True)
        return TrainState()
    accum = job.training.gradient_accumulation_steps
    if getattr(model_cfg, "memory_lb_mode", None) == "loss_free" and accum > 1:
        # one bias update per optimizer step: interval and warm-up are given in optimizer steps and count forwards
        # (uttt_llm/flame/train.py:282-292)
        model_cfg = model_cfg.replace(
            memory_loss_free_update_interval=model_cfg.memory_loss_free_update_interval * accum,
            memory_loss_free_warmup_steps=int(getattr(model_cfg, "memory_loss_free_warmup_steps", 0)) * accum)
    ecfg = EngineConfig(micro_batch_size=job.training.micro_batch_size or job.training.batch_size,
                        lr=job.optimizer.lr, eps=job.optimizer.eps, beta1=job.optimizer.beta1, beta2=job.optimizer.beta2,
                        weight_decay=job.optimizer.weight_decay, max_norm=job.training.max_norm,
                        warmup_steps=job.lr_scheduler.warmup_steps, total_steps=job.training.steps,
                        decay_type=job.lr_scheduler.decay_type, lr_min=job.lr_scheduler.lr_min,
                        skip_nan_inf=job.training.skip_nan_inf, seed=job.training.seed,
                        # The recompute of every (chunk, layer) region belongs to the model, as in the reference
                        # (modeling_recurrent_lact.py:3501 checkpoints unconditionally; its job files say
                        # mode = "none").  The job-level modes would wrap whole blocks on top of that, which
                        # recomputes nothing more: all three select the same schedule; `keep_layers` opts
                        # layers out of it where memory allows.
                        activation_checkpoint=True,
                        keep_activation_layers=tuple(int(i) for i in job.activation_checkpoint.keep_layers),
                        activation_offload=job.activation_offload.mode == "offload",
                        cuda_graph=bool(job.training.cuda_graph),
                        data_parallel_replicate_degree=int(job.training.data_parallel_replicate_degree),
                        shard_parameters=str(job.training.fsdp_reshard_after_forward) == "always")
    engine = TrainEngine(model_cfg, ecfg)
    if rank == 0 and job.job.print_args:
        print("\n".join(param_check(engine.model)), flush=True)
    if job.training.varlen:
        raise NotImplementedError("training.varlen: the chunk recurrence of these models has no per-document reset "
                                  "(documents are packed back to back, as in the reference's runs); the collator "
                                  "supports it for models that take cu_seqlens")
    t = job.training
    data = build_dataloader(t.dataset, vocab_size=model_cfg.vocab_size, seq_len=t.seq_len,
                            batch_size=t.batch_size * accum, rank=rank, world=world, seed=t.seed,
                            data_files=t.data_files, tokenizer_path=job.model.tokenizer_path or None,
                            dataset_name=t.dataset_name, dataset_split=t.dataset_split, data_dir=t.data_dir,
                            data_probs=t.data_probs, streaming=t.streaming, num_workers=t.num_workers,
                            prefetch_factor=t.prefetch_factor, pin_memory=t.pin_memory,
                            persistent_workers=t.persistent_workers, varlen=t.varlen, context_len=t.context_len)
    state = TrainState()
    ckpt = CheckpointManager(job.job.dump_folder, job.checkpoint.folder, job.checkpoint.interval,
                             job.checkpoint.keep_latest_k, job.checkpoint.save_backend,
                             job.checkpoint.model_weights_only, job.checkpoint.export_dtype,
                             job.checkpoint.enable_checkpoint, job.checkpoint.initial_load_path,
                             job.checkpoint.exclude_from_loading, job.checkpoint.async_mode)
    loaded = None
    if job.checkpoint.enable_checkpoint:
        loaded = ckpt.load(engine.model, engine.trainer, engine.lr_sched, data, state, step=job.checkpoint.load_step)
    if os.environ.get("TRAIN_ATTEMPT_KIND") == "resume" and loaded is None:
        raise RuntimeError("TRAIN_ATTEMPT_KIND=resume but no checkpoint could be loaded")
    if loaded:
        engine.step = state.step
        engine.lr_sched.fast_forward(state.step)
    if job.checkpoint.create_seed_checkpoint:
        ckpt.save(0, engine.model, engine.trainer, engine.lr_sched, data, state, force=True)
        return state
    n_params, flops_tok = get_nparams_and_flops(engine.model, model_cfg, job.training.seq_len)
    metrics = Metrics(job, rank, flops_tok, world)
    if rank == 0:
        print(f"model {model_cfg.model_type}: {n_params:,} parameters, {flops_tok / 1e9:.2f} GFLOP/token; "
              f"world {world}, global batch {job.training.batch_size * world * accum}", flush=True)
    prof = None
    if job.profiling.enable_profiling:
        from torch.profiler import ProfilerActivity, profile, schedule, tensorboard_trace_handler
        folder = os.path.join(job.job.dump_folder, job.profiling.save_traces_folder)
        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA],
                       schedule=schedule(wait=max(job.profiling.profile_freq - 2, 0), warmup=1, active=1),
                       on_trace_ready=tensorboard_trace_handler(folder))
        prof.start()
        from ..utils import trace
        trace.enable(True)            # named ranges per chunk / layer / write show up in the trace
    snapshot = bool(job.profiling.enable_memory_snapshot) and torch.cuda.is_available()
    if snapshot:
        torch.cuda.memory._record_memory_history(max_entries=100000)
    t0 = time.perf_counter()
    # garbage collection at fixed steps on every rank instead of whenever each interpreter feels like it: an
    # unsynchronised collection stalls one rank and with it every collective (training.gc_freq)
    gc_freq = int(job.training.gc_freq or 0)
    if gc_freq > 0:
        gc.disable()
        gc.collect(1)
    skipped_on_device = None          # running count of skipped steps, read back only when logging
    first_step = True
    while state.step < job.training.steps:
        # the step number as the model's statistics hooks see it (the pool statistics are taken every N steps)
        os.environ["FLAME_TRAIN_STEP"] = str(state.step + 1)
        batch = next(data)
        loss = engine.train_step(batch)
        state.step += 1
        state.token += batch["input_ids"].numel() * world
        stats = dict(engine.last_stats)
        skipped = stats["skipped"].detach().to(torch.int64) if torch.is_tensor(stats["skipped"]) \
            else torch.tensor(int(bool(stats["skipped"])))
        skipped_on_device = skipped if skipped_on_device is None else skipped_on_device + skipped
        logging_step = state.step % job.metrics.log_freq == 0 or state.step == 1
        saving_step = ckpt.should_save(state.step, state.step == job.training.steps and job.checkpoint.enable_checkpoint)
        if logging_step or saving_step:
            state.skipped_step += int(skipped_on_device.item())       # every skipped step since the last read
            skipped_on_device = None
            engine.check_kernel_status()                               # never log or save on top of a failed kernel
        metrics.log(state.step, loss, stats, batch["input_ids"].numel(), state)
        state.elapsed = time.perf_counter() - t0
        ckpt.save(state.step, engine.model, engine.trainer, engine.lr_sched, data, state,
                  force=state.step == job.training.steps and job.checkpoint.enable_checkpoint)
        if first_step:
            # start-up (lazy initialisation, first allocations) is over: a rank that stops answering now fails
            # the others' next collective after the training time-out, not the start-up one
            set_collective_timeout(job.comm.train_timeout_seconds)
            first_step = False
        if gc_freq > 0 and state.step % gc_freq == 0:
            gc.collect(1)
        if prof is not None:
            prof.step()
    ckpt.wait()
    if gc_freq > 0:
        gc.enable()
    if prof is not None:
        prof.stop()
    if snapshot:
        folder = os.path.join(job.job.dump_folder, job.profiling.save_memory_snapshot_folder)
        os.makedirs(folder, exist_ok=True)
        torch.cuda.memory._dump_snapshot(os.path.join(folder, f"rank{rank}_memory_snapshot.pickle"))
        torch.cuda.memory._record_memory_history(enabled=None)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return state


if __name__ == "__main__":
    main()
