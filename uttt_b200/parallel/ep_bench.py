"""Micro-benchmark of the fused compute + collective kernels (one process per GPU): expert-parallel dispatch /
combine and the all-gather-fused GEMM.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m uttt_b200.parallel.ep_bench [--batch 4] [--rows 8192] [--dim 384] [--experts 32] [--topk 2]

Times, with CUDA events on the device and the maximum over ranks: the fused peer-memory path (``ep_push`` /
``ep_pull`` kernels, including their ordering collectives and staging copies) and the all-to-all baseline (local
permute + ``all_to_all_single`` + local un-permute) on the same routing.  Prints one JSON line on rank 0 with the
bytes that cross NVLink per rank and the fraction of the measured 770 GB/s per-direction peer copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..utils.clocks import ClockSampler

from ..ops import functional as F_ops
from .expert_parallel import ExpertParallel


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _measured_tflops() -> float:
    for cand in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        try:
            with open(cand) as fh:
                return float(json.load(fh)["bf16_tflops"])
        except Exception:
            continue
    return 1590.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--rows", type=int, default=8192, help="rows per sequence (tokens x fast-weight heads)")
    ap.add_argument("--dim", type=int, default=384)
    ap.add_argument("--experts", type=int, default=32)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gather-ctas", type=int, default=24)
    args = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    sampler = ClockSampler(rank)          # SM clock and throttle reasons of this rank's GPU during the timings
    sampler.start()
    torch.manual_seed(7 + dist.get_rank())
    b, n, d, e, k = args.batch, args.rows, args.dim, args.experts, args.topk
    idx = torch.rand(b, n, e, device=dev).topk(k, dim=-1).indices
    plan = F_ops.build_group_plan(idx, e)
    rows = torch.randn(b * n, d, device=dev, dtype=torch.bfloat16)
    w = torch.rand(b * n, k, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {"n_gpus": world, "rows_per_rank": b * n, "dim": d, "experts": e, "topk": k}
    remote_frac = (world - 1) / world
    nvlink_bytes = b * n * k * d * 2 * remote_frac
    for name in ("peer", "a2a"):
        ep = ExpertParallel(None, dev, e, transport=name, max_row_bytes=4 * d)
        eplan = ep.plan(plan, idx)
        with torch.no_grad():
            xp = ep.dispatch(rows, None, eplan)
            t_plan = _time(lambda: ep.plan(plan, idx), args.iters, flush)
            t_disp = _time(lambda: ep.dispatch(rows, None, eplan), args.iters, flush)
            t_comb = _time(lambda: ep.combine(xp, w, eplan), args.iters, flush)
        extra = {}
        if name == "peer":
            # the NVLink kernels alone (no ordering collective, no staging copy): what the link sees
            from ..ops._ext import load
            ext = load(required=True)
            from .expert_parallel import _map_args
            cap = eplan.owner.rows_padded
            slot = ep._slot(ep._recv, "recv", cap, d, rows.dtype)
            ptrs = ep.heap.peer_ptrs(slot)
            t_push = _time(lambda: ext.ep_push(rows, None, *_map_args(eplan)[:3], eplan.sizes32, eplan.remote_start,
                                               ptrs, e, n, cap), args.iters, flush)
            t_pull = _time(lambda: ext.ep_pull(ptrs, w, *_map_args(eplan), e, n, d, rows.dtype, cap), args.iters,
                           flush)
            # the read of the pool through its owners: dispatch -> gate|up GEMM with SwiGLU -> down GEMM -> combine,
            # host-ordered (a scalar collective and a staging copy around each transfer) against the tile-driven
            # chain of four kernels (expert_parallel.py::fused_read)
            inter = 4 * d
            g_owner = eplan.owner.num_groups
            w02 = (torch.randn(g_owner, 2 * inter, d, device=dev) * 0.05).bfloat16()
            w1 = (torch.randn(g_owner, d, inter, device=dev) * 0.05).bfloat16()

            def read_ordered():
                xq = ep.dispatch(rows, None, eplan)
                hid = F_ops.gg_swiglu(xq, w02, eplan.owner)
                return ep.combine(F_ops.gg_nt(hid, w1, eplan.owner), w, eplan)

            def read_gemms_only():
                return F_ops.gg_nt(F_ops.gg_swiglu(xp, w02, eplan.owner), w1, eplan.owner)

            y_a = read_ordered()
            y_b = ep.fused_read(rows, w, w02, w1, eplan)
            rel = float((y_a.float() - y_b.float()).norm() / y_a.float().norm().clamp_min(1e-12))
            t_ordered = _time(read_ordered, args.iters, flush)
            t_fused = _time(lambda: ep.fused_read(rows, w, w02, w1, eplan), args.iters, flush)
            t_gemms = _time(read_gemms_only, args.iters, flush)
            # the four kernels of the tile-driven chain one by one (counters already satisfied, so nothing waits)
            tiles = cap // 128
            rdy, dne = ep._ready[0], ep._done[0]
            snd = ep._slot(ep._send, "send", cap, d, rows.dtype)
            full = torch.full_like(rdy, 1 << 30)
            hid0 = F_ops.gg_swiglu(xp, w02, eplan.owner)
            t_push_sig = _time(lambda: ext.ep_push(rows, None, *_map_args(eplan)[:3], eplan.sizes32,
                                                   eplan.remote_start, ptrs, e, n, cap, ep.heap.peer_ptrs(rdy)),
                               args.iters, flush)
            dist.barrier()
            rdy.zero_()
            t_up_flow = _time(lambda: ext.gg_nt_swiglu(slot, w02, eplan.owner.tile_group, full[:tiles], 128, 0.0),
                              args.iters, flush)
            t_up = _time(lambda: ext.gg_nt_swiglu(slot, w02, eplan.owner.tile_group), args.iters, flush)
            t_down_flow = _time(lambda: ext.gg_nt(hid0, w1, eplan.owner.tile_group, snd, None, 0, dne[:tiles], 0.0),
                                args.iters, flush)
            t_down = _time(lambda: ext.gg_nt(hid0, w1, eplan.owner.tile_group, snd), args.iters, flush)
            dist.barrier()
            t_pull_flow = _time(lambda: ext.ep_pull(ep.heap.peer_ptrs(snd), w, *_map_args(eplan), e, n, d, rows.dtype,
                                                    cap, ep.heap.peer_ptrs(dne), 1, 0.0), args.iters, flush)
            dist.barrier()
            for t in ep._done:
                t.zero_()
            ep._done_uses = [0, 0]
            dist.barrier()
            pieces = {"push_with_row_counts_ms": round(t_push_sig, 4), "push_plain_ms": round(t_push, 4),
                      "gate_up_gemm_with_tile_waits_ms": round(t_up_flow, 4), "gate_up_gemm_plain_ms": round(t_up, 4),
                      "down_gemm_with_tile_reports_ms": round(t_down_flow, 4), "down_gemm_plain_ms": round(t_down, 4),
                      "pull_with_tile_waits_ms": round(t_pull_flow, 4), "pull_plain_ms": round(t_pull, 4)}
            flops = 6.0 * b * n * k * d * inter
            peak = _measured_tflops()
            t_compute = flops / peak / 1e9
            t_link = 2.0 * nvlink_bytes / 770.0 / 1e6          # rows out and results back, per direction and rank
            status = int(ext.gemm_status(torch.zeros(1, device=dev))[0])
            extra_read = {"host_ordered_ms": round(t_ordered, 4), "tile_driven_ms": round(t_fused, 4),
                          "gemms_alone_ms": round(t_gemms, 4), "rel_diff_between_the_two": round(rel, 5),
                          "compute_at_measured_peak_ms": round(t_compute, 4),
                          "nvlink_at_measured_770GBs_ms": round(t_link, 4),
                          "tile_driven_roofline_frac": round(max(t_compute, t_link) / t_fused, 3),
                          "host_ordered_roofline_frac": round(max(t_compute, t_link) / t_ordered, 3),
                          "kernel_status": status, "kernels": pieces}
            out["read_through_owners"] = extra_read
            extra = {"push_kernel_ms": round(t_push, 4), "pull_kernel_ms": round(t_pull, 4),
                     "push_kernel_frac_of_measured_peer_copy": round(nvlink_bytes / t_push / 1e6 / 770.0, 3),
                     "pull_kernel_frac_of_measured_peer_copy": round(nvlink_bytes / t_pull / 1e6 / 770.0, 3)}
        out[name] = {**extra, "plan_ms": round(t_plan, 4), "dispatch_ms": round(t_disp, 4), "combine_ms": round(t_comb, 4),
                     "dispatch_gbs_per_rank": round(nvlink_bytes / t_disp / 1e6, 1),
                     "combine_gbs_per_rank": round(nvlink_bytes / t_comb / 1e6, 1),
                     "dispatch_frac_of_measured_peer_copy": round(nvlink_bytes / t_disp / 1e6 / 770.0, 3),
                     "combine_frac_of_measured_peer_copy": round(nvlink_bytes / t_comb / 1e6 / 770.0, 3)}
    # all-gather fused into the GEMM (weight rows sharded over the ranks) against all-gather + library GEMM
    from .ag_linear import ShardedWeightLinear
    from .symm import SymmetricHeap
    m_rows, k_in, n_out = 8192, 1536, 4096
    if n_out % (256 * world) == 0:
        heap = SymmetricHeap(dev, None, capacity_bytes=n_out * k_in * 2 + (1 << 20))
        layer = ShardedWeightLinear(heap, k_in, n_out, gather_ctas=args.gather_ctas)
        layer.load_full_weight(torch.randn(n_out, k_in, device=dev) / k_in ** 0.5)
        x = torch.randn(m_rows, k_in, device=dev, dtype=torch.bfloat16)
        full = torch.empty(n_out, k_in, device=dev, dtype=torch.bfloat16)
        shard = layer.shard.detach().clone()

        def baseline():
            dist.all_gather_into_tensor(full, shard)
            return x @ full.t()

        with torch.no_grad():
            t_fused = _time(lambda: layer(x), args.iters, flush)
            t_base = _time(baseline, args.iters, flush)
            t_gemm = _time(lambda: x @ full.t(), args.iters, flush)
        flops = 2.0 * m_rows * k_in * n_out
        out["ag_gemm"] = {"M": m_rows, "K": k_in, "N": n_out, "fused_ms": round(t_fused, 4),
                          "allgather_then_gemm_ms": round(t_base, 4), "library_gemm_only_ms": round(t_gemm, 4),
                          "fused_tflops": round(flops / t_fused / 1e9, 1),
                          "remote_bytes": int(n_out * k_in * 2 * remote_frac)}
    out["clocks"] = sampler.stop()          # every rank ends its own sampler
    if dist.get_rank() == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
