"""Headline benchmark: training tokens/s of the 760M uTTT-MoE language model at 32K context.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched under torchrun)

``--model`` selects one of the other named configurations instead (the headline stays the default):
``124M-uttt-moe`` and ``124M-uttt-dense`` (tokens/s at 32K context) and ``nvs-uttt-moe`` (view-synthesis training,
scenes/s at 256 x 256, 4 input + 2 target views).

Every rank trains on its own synthetic Zipf(1.1) sequences (weak scaling: ``--per-gpu-batch``
sequences of 32768 tokens per GPU and step, so 8 GPUs x 4 = the global batch of 32).  A step is
forward + backward over the rank's sequences, the gradient reduction, clipping, AdamW and the
parameter redistribution.  Two numbers are taken, both with CUDA events between
barrier + synchronize fences, max over ranks:

* ``value``: steps on batches already resident on the device (kernel-side throughput);
* ``e2e``: steps through ``TrainEngine.train_step`` from pinned host memory with the loss read
  back to the host every step.

``--impl reference`` runs the unmodified reference implementation from ``baseline/_ref`` on the
same metric and shape (see baseline/run_reference.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S = None      # the reference publishes no throughput number
METRIC_NAMES = {"760M-uttt-moe": "760M uTTT-MoE", "124M-uttt-moe": "124M uTTT-MoE", "124M-uttt-dense": "124M uTTT-Dense"}


from uttt_b200.utils.clocks import ClockSampler  # noqa: E402  (kept importable as bench.ClockSampler)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from uttt_b200 import ops
    from uttt_b200.config import named_config
    from uttt_b200.ops._ext import load
    from uttt_b200.train.data import SyntheticZipfTokens
    from uttt_b200.train.engine import EngineConfig, TrainEngine, init_distributed

    rank, world, local = init_distributed()
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    ext = load(required=True)
    ops.set_dense_gemm(args.dense_gemm == "own")
    ops.set_strict(True)          # a bf16 GPU tensor that leaves the extension's kernels raises instead of falling back
    dev = torch.device("cuda", local)
    over = dict(memory_update_backward_mode=args.backward_mode) if args.model != "124M-uttt-dense" else {}
    if args.expert_parallel > 1:
        over["memory_expert_parallel"] = args.expert_parallel
    cfg = named_config(args.model, **over)
    seq = args.seq_len
    keep_arg = args.keep_activation_layers
    if keep_arg == "auto":
        # two of the 24 layers keep their activations (about 18 GB each at 4 x 32K tokens): 140 GB peak on a 180 GB part
        keep_arg = "0,12" if (args.model == "760M-uttt-moe" and args.micro_batch * args.seq_len <= 4 * 32768) else ""
    keep = tuple(int(i) for i in keep_arg.split(",") if i.strip())
    eng = TrainEngine(cfg, EngineConfig(micro_batch_size=args.micro_batch, lr=1e-3, eps=1e-15, warmup_steps=1024,
                                        total_steps=40960, seed=42, keep_activation_layers=keep,
                                        cuda_graph=not args.no_cuda_graph and args.expert_parallel <= 1,
                                        expert_capacity_factor=float(min(max(args.expert_parallel, 2), 4))), dev)
    data = SyntheticZipfTokens(cfg.vocab_size, seq, args.per_gpu_batch, seed=1234, rank=rank, world=world)
    n_params = eng.trainer.num_parameters()

    def fence():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(step_fn, batches):
        fence()
        sampler = ClockSampler(local)
        sampler.start()
        launches0 = ops.launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for b in batches:
            step_fn(b)
        end.record()
        torch.cuda.synchronize(dev)
        launches = ops.launch_count() - launches0
        clocks = sampler.stop()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([start.elapsed_time(end) / len(batches)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), launches, clocks

    # warm-up (allocator, lazy tables, cuBLAS handles)
    for _ in range(max(args.warmup, 3)):
        float(eng.train_step(next(data)))
    # (1) device-resident batches: distinct inputs every step, working set per step >> L2
    dev_batches = [{k: v.to(dev) for k, v in next(data).items()} for _ in range(args.steps)]
    ms, launches, clocks = timed(lambda b: eng.train_step(b), dev_batches)
    # (2) end to end through the public API: pinned host batch -> device, loss -> host, every step
    host_batches = [next(data) for _ in range(args.steps)]
    losses = []
    ms_e2e, _, clocks_e2e = timed(lambda b: losses.append(float(eng.train_step(b))), host_batches)
    status = int(ext.gemm_status(torch.zeros(1, device=dev))[0])
    tokens_per_step = args.per_gpu_batch * seq * world
    h2d = host_batches[0]["input_ids"].numel() * host_batches[0]["input_ids"].element_size()
    out = None
    if rank == 0:
        peak_gb = torch.cuda.max_memory_allocated(dev) / 2 ** 30
        out = {
            "metric": f"train tokens/s, {METRIC_NAMES[args.model]} 32K ctx", "value": tokens_per_step / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (tokens_per_step / (ms / 1e3) / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16", "data": "synthetic Zipf(1.1) token ids, random-init weights",
            "impl": "uttt_b200",
            "config": {"model": args.model, "params": n_params, "global_batch": args.per_gpu_batch * world,
                       "per_gpu_batch": args.per_gpu_batch, "micro_batch": args.micro_batch, "seq_len": seq,
                       "parallelism": (f"fsdp{world}" if world > 1 else "single")
                       + (f"+ep{args.expert_parallel}" if args.expert_parallel > 1 else ""),
                       "backward_mode": args.backward_mode,
                       "activation_recompute": "per (chunk, layer) and per chunk write" + (
                           f"; layers {list(keep)} keep their activations" if keep else ""),
                       "cache": "inputs and per-step working set are far larger than L2 (no flush needed)",
                       "dense_gemm": args.dense_gemm,
                       "cuda_graph": ("forward + backward of a micro-batch replayed as one CUDA graph; optimizer eager"
                                      if eng._graphs else f"off ({eng.graph_error or 'not requested'})")},
            "clocks": clocks,
            "e2e": {"value": tokens_per_step / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "clocks": clocks_e2e,
                    "last_loss": losses[-1] if losses else None},
            "gpu_launches": launches, "peak_mem_gib": round(peak_gb, 2),
            "peak_reserved_gib": round(torch.cuda.max_memory_reserved(dev) / 2 ** 30, 2), "kernel_status": status,
        }
    eng.release_graphs()
    # extra key: the same step with the pool's experts sharded over all ranks (expert parallelism).  The headline run
    # above keeps every sequence's pool on its own rank, as the reference does.
    want_ep = (world > 1 and args.expert_parallel <= 1 and not args.no_ep_extra and args.model != "124M-uttt-dense"
               and cfg.memory_num_experts % world == 0)
    if want_ep:
        import gc
        import threading

        def give_up():
            # the extra measurement must never cost the headline line
            if out is not None:
                out["ep"] = {"unavailable": "the expert-parallel measurement did not finish within its time limit"}
                print(json.dumps(out), flush=True)
            sys.stdout.flush()
            os._exit(0)
        guard = threading.Timer(float(args.ep_extra_limit), give_up)
        guard.daemon = True
        guard.start()
        ep_line = None
        try:
            del eng
            gc.collect()
            torch.cuda.empty_cache()
            cfg_ep = named_config(args.model, **{**over, "memory_expert_parallel": world})
            eng = TrainEngine(cfg_ep, EngineConfig(micro_batch_size=args.micro_batch, lr=1e-3, eps=1e-15,
                                                   warmup_steps=1024, total_steps=40960, seed=42,
                                                   keep_activation_layers=keep,
                                                   # staging for up to four times the balanced share per owner
                                                   # (the worst case up to 4 ranks): a random-init router sends a
                                                   # quarter of the experts more than twice their share
                                                   expert_capacity_factor=float(min(world, 4))), dev)
            for _ in range(2):
                float(eng.train_step(next(data)))
            ep_batches = [{k: v.to(dev) for k, v in next(data).items()} for _ in range(2)]
            ms_ep, launches_ep, clocks_ep = timed(lambda b: eng.train_step(b), ep_batches)
            ep_line = {"value": tokens_per_step / (ms_ep / 1e3), "unit": "tokens/s", "ms_per_step": ms_ep, "steps": 2,
                       "warmup": 2, "expert_parallel": world, "vs_expert_parallel_off": ms / ms_ep,
                       "read_path": "host-ordered dispatch / combine (autograd records every training forward; "
                                    "the tile-driven read serves forwards without autograd)",
                       "kernel_status": int(ext.gemm_status(torch.zeros(1, device=dev))[0]), "clocks": clocks_ep,
                       "gpu_launches": launches_ep}
            if ep_line["kernel_status"] != 0:
                # after a reported overflow or a failed wait the tensor-core kernels return at once: no valid timing
                ep_line = {"unavailable": f"device status word {ep_line['kernel_status']} during the "
                                          f"expert-parallel steps (61 = staging overflow, 6x = a bounded wait ran out)"}
        except Exception as exc:                       # e.g. out of memory: report, keep the headline
            ep_line = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        guard.cancel()
        if out is not None:
            out["ep"] = ep_line
    if out is not None:
        print(json.dumps(out), flush=True)
    _leave(world)


def _leave(world: int) -> None:
    """Leave the process group.  The result line is out already; if tearing the communicators down does not return
    within half a minute the process exits anyway (a wedged teardown must not turn a finished run into a time-out)."""
    if world <= 1:
        return
    import threading
    import torch.distributed as dist
    dist.barrier()

    def _teardown():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
    t = threading.Thread(target=_teardown, daemon=True)
    t.start()
    t.join(30.0)
    if t.is_alive():
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_nvs(args):
    """View-synthesis training throughput (scenes/s): LVSM-style decoder with a shared 16-expert pool, 256 x 256
    views patchified 8 x 8, 4 posed input views then 2 target views per scene, MSE loss, 16 scenes per GPU and step
    (8 GPUs = the global batch of 128), synthetic scenes (smoothed noise images, cameras on a radius-2 sphere)."""
    import torch
    import torch.distributed as dist
    from uttt_b200 import ops
    from uttt_b200.nvs.data import SyntheticScenes
    from uttt_b200.nvs.trainer import NVSTrainer, load_config
    from uttt_b200.ops._ext import load
    from uttt_b200.train.engine import init_distributed

    rank, world, local = init_distributed()
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    ext = load(required=True)
    dev = torch.device("cuda", local)
    cfg = load_config(os.path.join(ROOT, "configs", "nvs", "named", "uttt_moe_256_4in2out.yaml"))
    autoregressive = args.model == "nvs-uttt-moe-ar"
    if autoregressive:
        # the reference's stock layout: every view but the last is an input, every view but the first a target
        # (2 x 5 view slots of 1024 tokens for 6 views); this is the shape its own model can run
        cfg["model"]["view_layout"] = "autoregressive"
        cfg["model"].pop("num_input_views", None)
    per_gpu = args.per_gpu_batch if args.per_gpu_batch != 4 else 16
    cfg["training"].update(batch_size_per_gpu=per_gpu, total_batch_size=per_gpu * world, out_dir="/tmp/uttt_nvs_bench",
                           checkpoint_every=10 ** 9, print_every=10 ** 9, warmup=0, cuda_graph=not args.no_cuda_graph)
    trainer = NVSTrainer(cfg, device=dev)
    views, size = int(cfg["training"]["num_views"]), int(cfg["model"]["image_size"])
    data = SyntheticScenes(per_gpu, views, size, seed=1234, rank=rank)

    def fence():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(step_fn, batches):
        fence()
        sampler = ClockSampler(local)
        sampler.start()
        launches0 = ops.launch_count()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for b in batches:
            step_fn(b)
        end.record()
        torch.cuda.synchronize(dev)
        launches = ops.launch_count() - launches0
        clocks = sampler.stop()
        ms = torch.tensor([start.elapsed_time(end) / len(batches)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), launches, clocks

    for _ in range(max(args.warmup, 3)):
        float(trainer.train_pass(next(data))["loss"])
    dev_batches = [{k: v.to(dev) for k, v in next(data).items()} for _ in range(args.steps)]
    ms, launches, clocks = timed(lambda b: trainer.train_pass(b), dev_batches)
    host_batches = [next(data) for _ in range(args.steps)]
    losses = []
    ms_e2e, _, clocks_e2e = timed(lambda b: losses.append(float(trainer.train_pass(b)["loss"])), host_batches)
    status = int(ext.gemm_status(torch.zeros(1, device=dev))[0])
    scenes = per_gpu * world
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
    if rank == 0:
        print(json.dumps({
            "metric": ("train scenes/s, NVS uTTT-MoE 256x256, 6 views per scene in the reference's stock layout"
                       if autoregressive else "train scenes/s, NVS uTTT-MoE 256x256, 4 input + 2 target views"),
            "value": scenes / (ms / 1e3),
            "unit": "scenes/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic scenes (smoothed Gaussian-noise images, cameras on a radius-2 sphere, FOV 50)",
            "impl": "uttt_b200",
            "config": {"model": args.model + " (24 layers, d 768, 12 heads, 16 experts, top-2)",
                       "params": trainer.trainer.num_parameters(), "global_batch": scenes, "per_gpu_batch": per_gpu,
                       "views": views, "tokens_per_scene": (2 * (views - 1) if autoregressive else views) * (size // 8) ** 2,
                       "parallelism": f"dp{world}" if world > 1 else "single",
                       "cache": "inputs and per-step working set are far larger than L2 (no flush needed)",
                       "cuda_graph": ("forward + backward replayed as one CUDA graph; optimizer eager"
                                      if trainer._graphs else f"off ({trainer.graph_error or 'not requested'})")},
            "clocks": clocks,
            "e2e": {"value": scenes / (ms_e2e / 1e3), "unit": "scenes/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "clocks": clocks_e2e,
                    "last_loss": losses[-1] if losses else None},
            "gpu_launches": launches, "peak_mem_gib": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2),
            "kernel_status": status}), flush=True)
    trainer.release_graphs()
    _leave(world)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="760M-uttt-moe",
                    choices=["760M-uttt-moe", "124M-uttt-moe", "124M-uttt-dense", "nvs-uttt-moe", "nvs-uttt-moe-ar"])
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--per-gpu-batch", type=int, default=4)
    ap.add_argument("--micro-batch", type=int, default=int(os.environ.get("UTTT_BENCH_MICRO_BATCH", "4")))
    ap.add_argument("--backward-mode", default="full")
    ap.add_argument("--no-ep-extra", action="store_true",
                    help="skip the extra expert-parallel measurement that multi-GPU runs add under the key 'ep'")
    ap.add_argument("--ep-extra-limit", type=float, default=300.0, help="seconds allowed for that measurement")
    ap.add_argument("--dense-gemm", default="library", choices=["library", "own"],
                    help="dense projections on cuBLAS (default) or on the batched tcgen05 kernel of this repository")
    ap.add_argument("--no-cuda-graph", action="store_true",
                    help="launch every kernel of forward + backward from the host instead of replaying a CUDA graph")
    ap.add_argument("--keep-activation-layers", default=os.environ.get("UTTT_BENCH_KEEP_LAYERS", "auto"),
                    help="comma-separated layer indices whose activations are kept instead of recomputed")
    ap.add_argument("--expert-parallel", type=int, default=1,
                    help="shard the experts of the pool over this many ranks (default: pool state stays with its "
                         "sequence's rank, as in the reference)")
    args = ap.parse_args()
    if args.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(args)
    elif args.model in ("nvs-uttt-moe", "nvs-uttt-moe-ar"):
        run_nvs(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
