"""Resume with more than one rank: every rank continues its OWN data stream where it stopped."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, folder: str, out_path: str):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from uttt_b200.config import named_config
    from uttt_b200.train.checkpoint import CheckpointManager, TrainState
    from uttt_b200.train.data import SyntheticZipfTokens
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    cfg = named_config("tiny-uttt-moe")
    device = torch.device("cpu")

    def fresh():
        eng = TrainEngine(cfg, EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0), device)
        data = SyntheticZipfTokens(cfg.vocab_size, 128, 2, seed=7, rank=rank, world=world, pin=False)
        return eng, data

    # uninterrupted run: 3 steps, remember the 4th batch of this rank
    eng, data = fresh()
    for _ in range(3):
        eng.train_step(next(data))
    want_next = next(data)["input_ids"].clone()
    # interrupted run: 3 steps, save, rebuild everything, load
    eng, data = fresh()
    for _ in range(3):
        eng.train_step(next(data))
    ckpt = CheckpointManager(folder, interval=1, keep_latest_k=0)
    state = TrainState(step=3)
    ckpt.save(3, eng.model, eng.trainer, eng.lr_sched, data, state)
    eng2, data2 = fresh()
    loaded = ckpt.load(eng2.model, eng2.trainer, eng2.lr_sched, data2, TrainState())
    got_next = next(data2)["input_ids"]
    # a checkpoint written by fewer ranks has no entry for this rank: that must be an error, not a silent restart
    flat = ckpt._dcp_load(ckpt.path(3))
    both = "dataloader.rank_0" in flat and "dataloader.rank_1" in flat
    torch.save({"loaded": loaded, "same": bool(torch.equal(got_next, want_next)), "both_ranks_saved": both},
               f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_resume_continues_each_ranks_data(tmp_path):
    port = _free_port()
    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, port, str(tmp_path / "run"), out), nprocs=2, join=True)
    for rank in range(2):
        res = torch.load(f"{out}.{rank}")
        assert res["loaded"] == 3 and res["both_ranks_saved"]
        assert res["same"], f"rank {rank} did not continue its data stream after the resume"


def test_missing_rank_entry_is_an_error(tmp_path):
    """Single process stands in for 'rank 1 of a job resumed from a 1-rank checkpoint'."""
    import pytest
    sys.path.insert(0, ROOT)
    from uttt_b200.config import named_config
    from uttt_b200.train import checkpoint as ck
    from uttt_b200.train.data import SyntheticZipfTokens
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    cfg = named_config("tiny-uttt-moe")
    eng = TrainEngine(cfg, EngineConfig(micro_batch_size=2, warmup_steps=0, total_steps=4), torch.device("cpu"))
    data = SyntheticZipfTokens(cfg.vocab_size, 128, 2, seed=7, pin=False)
    mgr = ck.CheckpointManager(str(tmp_path), interval=1)
    mgr.save(1, eng.model, eng.trainer, eng.lr_sched, data, ck.TrainState(step=1))
    orig = ck._rank
    ck._rank = lambda: 1
    try:
        with pytest.raises(ck.MissingRankState):
            mgr.load(eng.model, eng.trainer, eng.lr_sched, data, ck.TrainState())
    finally:
        ck._rank = orig
