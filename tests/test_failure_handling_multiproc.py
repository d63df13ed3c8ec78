"""Failure handling across ranks, injected on the host only (gloo ranks on CPU; no device is ever faulted):

* a NaN loss on ONE rank makes EVERY rank skip the optimizer step (the gradient norm is a collective quantity and
  the skip is decided from it on the device), parameters and moments stay untouched, the next clean step applies;
* a rank that leaves between steps makes the survivors' next collective raise within the process-group timeout
  instead of hanging.
"""
import datetime
import os
import socket
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg():
    from uttt_b200.config import named_config
    return named_config("tiny-uttt-moe", hidden_size=128, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                        memory_num_active_experts=2, chunk_size=64, window_size=64)


def _nan_worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    eng = TrainEngine(_cfg(), EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0),
                      torch.device("cpu"))
    g = torch.Generator().manual_seed(7 + rank)
    ids = torch.randint(0, 1024, (2, 128), generator=g)
    batch = {"input_ids": ids, "labels": ids}
    eng.train_step(batch)                                            # a clean step
    before = {k: v.detach().clone() for k, v in eng.model.state_dict().items() if v.is_floating_point()}
    inner_forward = eng.model.forward

    def poisoned(*a, **k):                                           # host-side injection: rank 1 produces a NaN loss
        out = inner_forward(*a, **k)
        if rank == 1:
            out.loss = out.loss * float("nan")
        return out

    eng.model.forward = poisoned
    eng.train_step(batch)
    skipped = bool(eng.last_stats["skipped"])
    unchanged = all(torch.equal(before[k], v) for k, v in eng.model.state_dict().items() if k in before)
    eng.model.forward = inner_forward
    eng.train_step(batch)                                            # training continues
    moved = any(not torch.equal(before[k], v) for k, v in eng.model.state_dict().items() if k in before)
    finite = all(torch.isfinite(v).all() for v in eng.model.state_dict().values() if v.is_floating_point())
    torch.save({"skipped": skipped, "unchanged": unchanged, "moved": moved, "finite": finite},
               os.path.join(out_dir, f"nan{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_nan_on_one_rank_skips_the_step_on_every_rank(tmp_path):
    mp.spawn(_nan_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        got = torch.load(tmp_path / f"nan{rank}.pt")
        assert got == {"skipped": True, "unchanged": True, "moved": True, "finite": True}, (rank, got)


def _leaver_worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)                                               # one healthy collective
    if rank == world - 1:
        # this rank leaves between steps, with nothing in flight
        os._exit(0)
    start = time.time()
    raised = ""
    try:
        dist.all_reduce(t)
    except Exception as exc:                                         # the survivors must get an error, not a hang
        raised = type(exc).__name__
    torch.save({"raised": raised, "seconds": time.time() - start}, os.path.join(out_dir, f"leave{rank}.pt"))
    os._exit(0)


def test_rank_that_leaves_between_steps_is_noticed_within_the_timeout(tmp_path):
    ctx = mp.spawn(_leaver_worker, args=(3, _free_port(), str(tmp_path)), nprocs=3, join=False)
    deadline = time.time() + 60
    while time.time() < deadline and not all((tmp_path / f"leave{r}.pt").exists() for r in range(2)):
        time.sleep(0.2)
    for p in ctx.processes:
        p.join(timeout=5)
        if p.is_alive():
            p.terminate()
    for rank in range(2):
        got = torch.load(tmp_path / f"leave{rank}.pt")
        assert got["raised"], "the collective returned although a rank had left"
        assert got["seconds"] < 30, got
