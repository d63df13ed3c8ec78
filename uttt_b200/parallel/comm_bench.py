"""Micro-benchmark of the sharded optimizer step's collectives (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m uttt_b200.parallel.comm_bench [--numel 28350000] [--iters 10]

For one flat unit of ``numel`` bf16 elements (default: one 760M block, 28.35 M parameters) it times, with CUDA
events on the device and the maximum over ranks:

* gradient reduce-scatter + scale + squared norm: the peer-pointer kernel (``rs_sumsq``, every rank loads its
  shard from each peer), the same kernel in its ``multimem.ld_reduce`` form (sum formed inside NVSwitch) and the
  library baseline (``reduce_scatter_tensor`` on an fp32 copy, scale, squared norm);
* AdamW on the shard + cast + all-gather: the peer-pointer kernel (``adamw_scatter``), its ``multimem.st`` form
  and the library baseline (``adamw_flat`` on the shard followed by ``all_gather_into_tensor``).

Prints one JSON line on rank 0.  NVLink bytes into (reduce) or out of (gather) one GPU and the fraction of the
measured 770 GB/s per-direction peer copy are given for the peer-pointer forms.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..utils.clocks import ClockSampler

from .symm import SymmetricHeap

PEER_GBS = 770.0


def _time(fn, iters, heap):
    for _ in range(3):
        fn()
    total = 0.0
    for _ in range(iters):
        heap.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return round(float(t), 4)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--numel", type=int, default=28_350_000)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    rank = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    sampler = ClockSampler(rank)          # SM clock and throttle reasons of this rank's GPU during the timings
    sampler.start()
    chunk = 1024 * world
    n = (args.numel + chunk - 1) // chunk * chunk
    shard = n // world
    lo = rank * shard
    heap = SymmetricHeap(dev, None, capacity_bytes=4 * n + (1 << 20), use_multimem=True)
    ext = heap.ext
    grad = heap.alloc(n, torch.bfloat16)
    comp = heap.alloc(n, torch.bfloat16)
    torch.manual_seed(1 + rank)
    grad.copy_(torch.randn(n, device=dev) * 0.01)
    comp.zero_()
    out = torch.empty(shard, dtype=torch.float32, device=dev)
    sq = torch.zeros(1, device=dev)
    p = torch.randn(shard, device=dev)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    one = torch.ones(1, device=dev)
    res = {"n_gpus": world, "numel": n, "multimem": heap.use_multimem}

    def rs(mc):
        ext.rs_sumsq(heap.peer_ptrs(grad), rank, lo, out, 1.0 / world, sq, True, mc)

    def rs_lib():
        g32 = grad.float()
        dist.reduce_scatter_tensor(out, g32)
        out.mul_(1.0 / world)
        sq.add_(out.pow(2).sum())

    def ad(mc):
        ext.adamw_scatter(p, out, m, v, heap.peer_ptrs(comp), rank, lo, True, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, one, one,
                          shard, mc)

    def ad_lib():
        ext.adamw_flat(p, out, m, v, comp[lo:lo + shard], 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, one, one, 1.0, shard)
        dist.all_gather_into_tensor(comp, comp[lo:lo + shard].clone())

    res["rs_peer_ms"] = _time(lambda: rs(0), args.iters, heap)
    res["rs_library_ms"] = _time(rs_lib, args.iters, heap)
    res["adamw_gather_peer_ms"] = _time(lambda: ad(0), args.iters, heap)
    res["adamw_gather_library_ms"] = _time(ad_lib, args.iters, heap)
    if heap.use_multimem:
        res["rs_multimem_ms"] = _time(lambda: rs(heap.multicast_addr(grad)), args.iters, heap)
        res["adamw_gather_multimem_ms"] = _time(lambda: ad(heap.multicast_addr(comp)), args.iters, heap)
    link_bytes = shard * 2 * (world - 1)
    res["nvlink_bytes_per_gpu"] = link_bytes
    for key in ("rs_peer_ms", "adamw_gather_peer_ms"):
        res[key.replace("_ms", "_frac_of_770GBs")] = round(link_bytes / (res[key] * 1e-3) / 1e9 / PEER_GBS, 3)
    res["clocks"] = sampler.stop()          # every rank ends its own sampler
    if rank == 0:
        print(json.dumps(res))
    heap.barrier()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
