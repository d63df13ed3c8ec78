"""Sharded optimizer engine across ranks: two gloo ranks on CPU must reproduce a single-process step on the
concatenated batch; on a multi-GPU box the same check runs over NCCL with the fused peer-memory kernels."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _batch(rank: int, seq: int = 128):
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 1024, (2, seq), generator=g)
    return {"input_ids": ids, "labels": ids}


def _cfg():
    from uttt_b200.config import named_config
    return named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                        memory_num_active_experts=2, chunk_size=64, window_size=64, memory_lb_loss_alpha=0.0)


def _worker(rank: int, world: int, port: int, backend: str, out_path: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    if backend == "nccl":
        os.environ["NCCL_NVLS_ENABLE"] = "0"
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        device = torch.device("cuda", rank)
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        device = torch.device("cpu")
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(_cfg(), EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0,
                                           weight_decay=0.1, eps=1e-3), device)
    losses = [float(eng.train_step(_batch(rank))) for _ in range(2)]
    fused = eng.trainer.symm is not None
    sd = {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}
    opt = eng.trainer.optimizer_state_dict()
    if rank == 0:
        torch.save({"model": sd, "losses": losses, "fused": fused,
                    "m": {k: v["exp_avg"] for k, v in opt["state"].items()}}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def _hybrid_worker(rank: int, world: int, port: int, replicas: int, out_path: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(_cfg(), EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0,
                                           weight_decay=0.1, eps=1e-3, data_parallel_replicate_degree=replicas),
                      torch.device("cpu"))
    assert eng.trainer.world == world // replicas and eng.trainer.replicas == replicas
    stats = None
    for _ in range(2):
        eng.train_step(_batch(rank))
        stats = eng.last_stats
    sd = {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}
    torch.save({"model": sd, "grad_norm": float(stats["grad_norm"]),
                "master_numel": sum(u.master.numel() for u in eng.trainer.units)}, out_path + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_hybrid_sharding_matches_full_sharding(tmp_path):
    """Four gloo ranks as 2 shard groups x 2 replicas (optimizer state sharded over two ranks, gradients all-reduced
    across the two replicas of each shard) train exactly like four ranks that shard over all of them."""
    runs = {}
    for replicas in (1, 2):
        out = str(tmp_path / f"h{replicas}.pt")
        mp.spawn(_hybrid_worker, args=(4, _free_port(), replicas, out), nprocs=4, join=True)
        runs[replicas] = [torch.load(out + f".{r}", weights_only=False) for r in range(4)]
    for r in range(4):                                   # every rank ends with the same parameters
        for k, v in runs[2][0]["model"].items():
            if v.is_floating_point():
                torch.testing.assert_close(runs[2][r]["model"][k], v, atol=0, rtol=0, msg=f"rank {r}: {k}")
    ratio = runs[2][0]["master_numel"] / runs[1][0]["master_numel"]          # shards are twice as large (up to padding)
    assert 1.95 < ratio < 2.05, ratio
    assert abs(runs[2][0]["grad_norm"] - runs[1][0]["grad_norm"]) <= 1e-5 * runs[1][0]["grad_norm"]
    for k, v in runs[1][0]["model"].items():
        if v.is_floating_point() and "loss_free" not in k:
            torch.testing.assert_close(runs[2][0]["model"][k], v, atol=2e-5, rtol=2e-4, msg=k)


def _sharded_param_worker(rank: int, world: int, port: int, shard: bool, out_path: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(_cfg(), EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0,
                                           weight_decay=0.1, eps=1e-3, shard_parameters=shard), torch.device("cpu"))
    released = []
    for _ in range(2):
        eng.train_step(_batch(rank))
        released.append(all(u.compute.untyped_storage().size() == 0 for u in eng.trainer.units))
    eval_loss = float(eng.eval_loss(_batch(0)))                 # gathers through the forward pre-hook
    sd = {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}
    torch.save({"model": sd, "released": released, "eval": eval_loss}, out_path + f".{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_parameter_shards_between_steps_train_like_full_buffers(tmp_path):
    """``shard_parameters`` (``training.fsdp_reshard_after_forward = "always"``): after a step each rank holds only its
    shard of the parameters (the full buffers have no storage), the next forward / state_dict gathers them, and
    training is bit-identical to keeping the full buffers."""
    runs = {}
    for shard in (False, True):
        out = str(tmp_path / f"s{int(shard)}.pt")
        mp.spawn(_sharded_param_worker, args=(2, _free_port(), shard, out), nprocs=2, join=True)
        runs[shard] = [torch.load(out + f".{r}", weights_only=False) for r in range(2)]
    assert runs[True][0]["released"] == [True, True] and runs[False][0]["released"] == [False, False]
    for r in range(2):
        assert runs[True][r]["eval"] == runs[False][r]["eval"]
        for k, v in runs[False][r]["model"].items():
            torch.testing.assert_close(runs[True][r]["model"][k], v, atol=0, rtol=0, msg=k)


def _single_process_reference(device: str, dtype_note: str):
    sys.path.insert(0, ROOT)
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(_cfg(), EngineConfig(micro_batch_size=4, lr=1e-2, warmup_steps=0, total_steps=10, seed=0,
                                           weight_decay=0.1, eps=1e-3), torch.device(device))
    both = {k: torch.cat([_batch(0)[k], _batch(1)[k]]) for k in ("input_ids", "labels")}
    for _ in range(2):
        eng.train_step(both)
    return {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()}


def test_two_gloo_ranks_match_single_process(tmp_path):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), "gloo", out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    want = _single_process_reference("cpu", "fp32")
    for k, v in want.items():
        if v.is_floating_point() and "loss_free" not in k:
            torch.testing.assert_close(got["model"][k], v, atol=2e-5, rtol=2e-4, msg=k)


@pytest.mark.gpu
def test_two_gpu_ranks_fused_kernels_match_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), "nccl", out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    assert got["fused"], "the peer-memory gradient path was not used"
    want = _single_process_reference("cuda", "bf16")
    worst = 0.0
    for k, v in want.items():
        if v.is_floating_point() and "loss_free" not in k:
            err = (got["model"][k] - v).abs().max().item()
            worst = max(worst, err)
            assert err < 3e-2, (k, err)      # bf16 parameters after two lr=1e-2 steps
    assert all(l == l for l in got["losses"])


def _ag_worker(rank: int, world: int, port: int, out_path: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uttt_b200.ops._ext import load
    from uttt_b200.parallel.ag_linear import ShardedWeightLinear
    from uttt_b200.parallel.symm import SymmetricHeap
    n, k, m = 1024, 384, 512
    heap = SymmetricHeap(dev, None, capacity_bytes=n * k * 2 + (1 << 20))
    layer = ShardedWeightLinear(heap, k, n, gather_ctas=8)
    g = torch.Generator(device="cpu").manual_seed(5)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(dev)
    layer.load_full_weight(w)
    torch.manual_seed(10 + rank)
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16, requires_grad=True)
    ok = True
    for _ in range(2):                                   # the second call re-gathers over the first call's copies
        y = layer(x)
        want = x.detach().float() @ w.bfloat16().float().t()
        ok = ok and bool(torch.allclose(y.float(), want, atol=3e-2, rtol=3e-2))
    gy = torch.randn_like(y)
    y.backward(gy)
    dx_want = gy.float() @ w.bfloat16().float()
    ok = ok and bool(torch.allclose(x.grad.float(), dx_want, atol=5e-2, rtol=5e-2))
    dw = gy.float().t() @ x.detach().float()
    dist.all_reduce(dw)
    rows = n // world
    ok = ok and bool(torch.allclose(layer.shard.grad.float(), dw[rank * rows:(rank + 1) * rows], atol=0.3, rtol=5e-2))
    status = int(load().gemm_status(x)[0])
    flag = torch.tensor([1.0 if (ok and status == 0) else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": bool(flag.item() == 1.0), "status": status}, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_all_gather_fused_gemm(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "ag.pt")
    mp.spawn(_ag_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    assert got["status"] == 0 and got["ok"]


def _multimem_worker(rank: int, world: int, port: int, out_path: str):
    """Switch-side reduction / broadcast forms of the optimizer-step kernels against the peer-pointer forms."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from uttt_b200.parallel.symm import SymmetricHeap
    n = 1 << 24                                           # elements per buffer, shard = n / world
    heap = SymmetricHeap(dev, None, capacity_bytes=n * (2 + 4 + 2 + 4) + (1 << 20), use_multimem=True)
    result = {"supported": heap.use_multimem}
    if heap.use_multimem:                                 # same answer on every rank: one fabric
        ext = heap.ext
        shard = n // world
        lo = rank * shard
        ok = True
        times = {}
        for dtype in (torch.bfloat16, torch.float32):
            grad = heap.alloc(n, dtype)
            comp = heap.alloc(n, dtype)
            torch.manual_seed(3 + rank)
            grad.copy_(torch.randint(-8, 9, (n,), device=dev).to(dtype) * 0.25)   # sums are exact in bf16
            comp.zero_()
            heap.barrier()
            outs = []
            for mc in (0, heap.multicast_addr(grad)):
                out = torch.empty(shard, dtype=torch.float32, device=dev)
                sq = torch.zeros(1, device=dev)
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                for it in range(4):
                    if it == 3:
                        ev[0].record()
                    sq.zero_()
                    ext.rs_sumsq(heap.peer_ptrs(grad), rank, lo, out, 0.5, sq, dtype == torch.bfloat16, mc)
                ev[1].record()
                torch.cuda.synchronize()
                times[f"rs_{'mc' if mc else 'peer'}_{str(dtype)[6:]}"] = ev[0].elapsed_time(ev[1])
                outs.append((out, sq.clone()))
            ok = ok and bool(torch.equal(outs[0][0], outs[1][0])) and bool(
                torch.allclose(outs[0][1], outs[1][1], rtol=1e-5))
            heap.barrier()
            # optimizer step + broadcast: the two forms must leave identical buffers on every rank
            g = outs[0][0]
            one = torch.ones(1, device=dev)
            got = []
            for mc in (0, heap.multicast_addr(comp)):
                p = torch.full((shard,), 0.5, device=dev)
                m = torch.zeros_like(p)
                v = torch.zeros_like(p)
                comp.zero_()
                heap.barrier()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
                ev[0].record()
                ext.adamw_scatter(p, g, m, v, heap.peer_ptrs(comp), rank, lo, dtype == torch.bfloat16, 1e-2, 0.9, 0.95,
                                  1e-8, 0.1, 1, one, one, shard, mc)
                ev[1].record()
                heap.barrier()
                torch.cuda.synchronize()
                times[f"adamw_{'mc' if mc else 'peer'}_{str(dtype)[6:]}"] = ev[0].elapsed_time(ev[1])
                got.append(comp.clone())
                heap.barrier()
            ok = ok and bool(torch.equal(got[0], got[1])) and bool((got[0] != 0).all())
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        result.update(ok=bool(flag.item() == 1.0), times=times)
    if rank == 0:
        torch.save(result, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_multimem_forms_match_peer_forms(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "mm.pt")
    mp.spawn(_multimem_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    if not got["supported"]:
        pytest.skip("the symmetric allocation has no multicast mapping on this box")
    print("multimem timings (ms):", got["times"])
    assert got["ok"]
