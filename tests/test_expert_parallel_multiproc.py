"""Expert-parallel pool: two ranks that shard the experts must reproduce the data-parallel run.

On CPU the ranks talk over gloo with the all-to-all transport; on a box with two GPUs the same check runs
over NCCL with the peer-memory dispatch / combine kernels (NVLS off, plain peer loads and stores)."""
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


def _cfg(ep: int, **over):
    from uttt_b200.config import named_config
    return named_config("tiny-uttt-moe", hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4,
                        memory_num_active_experts=2, chunk_size=64, window_size=64, memory_lb_loss_alpha=0.01,
                        memory_expert_parallel=ep, **over)


def _worker(rank: int, world: int, port: int, backend: str, out_dir: str, over=None):
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
    g = torch.Generator().manual_seed(100 + rank)
    ids = torch.randint(0, 1024, (2, 192), generator=g)
    batch = {"input_ids": ids, "labels": ids}
    result = {}
    for ep in (1, 2):
        eng = TrainEngine(_cfg(ep, **(over or {})), EngineConfig(micro_batch_size=2, lr=1e-2, warmup_steps=0, total_steps=10, seed=0,
                                                 weight_decay=0.0, eps=1e-3), device)
        # evaluation first, on the initial weights and without autograd: the write path then issues its three
        # dispatches (keys, values, learning rates) back to back before any of them is consumed
        eval_loss = float(eng.eval_loss(batch))
        losses = [float(eng.train_step(batch)) for _ in range(2)]
        result[ep] = {"losses": losses, "eval_loss": eval_loss,
                      "model": {k: v.detach().float().cpu() for k, v in eng.model.state_dict().items()},
                      "transport": None if eng.expert_parallel is None else eng.expert_parallel.transport}
    torch.save(result, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _check(out_dir, atol, rtol, want_transport):
    for rank in range(2):
        got = torch.load(os.path.join(out_dir, f"r{rank}.pt"), weights_only=False)
        assert got[2]["transport"] == want_transport
        a, b = got[1]["eval_loss"], got[2]["eval_loss"]
        assert abs(a - b) <= atol + rtol * abs(a), ("no_grad forward", a, b)
        for a, b in zip(got[1]["losses"], got[2]["losses"]):
            assert abs(a - b) <= atol + rtol * abs(a), (got[1]["losses"], got[2]["losses"])
        for k, v in got[1]["model"].items():
            if v.is_floating_point() and "loss_free" not in k:
                torch.testing.assert_close(got[2]["model"][k], v, atol=atol, rtol=rtol, msg=k)


def test_two_gloo_ranks_expert_parallel_matches_data_parallel(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), "gloo", str(tmp_path)), nprocs=2, join=True)
    _check(str(tmp_path), 3e-5, 3e-4, "a2a")


def test_two_gloo_ranks_expert_parallel_with_chained_writes(tmp_path):
    """Every writer layer applies its own update to the sharded bank in turn (no aggregate): the owners gather the
    momentum gates of all sequences of the group, as for the aggregated write."""
    mp.spawn(_worker, args=(2, _free_port(), "gloo", str(tmp_path), dict(memory_update_aggregate_write=False, memory_aggregate_momentum_mode="none")),
             nprocs=2, join=True)
    _check(str(tmp_path), 3e-5, 3e-4, "a2a")


def test_two_gloo_ranks_expert_parallel_with_cross_layer_cut(tmp_path):
    """Per-reader streams of the bank (each reader's gradient reaches only its own writer) over sharded experts."""
    mp.spawn(_worker, args=(2, _free_port(), "gloo", str(tmp_path), dict(memory_update_backward_mode="cross_layer_cut")),
             nprocs=2, join=True)
    _check(str(tmp_path), 3e-5, 3e-4, "a2a")


@pytest.mark.gpu
@pytest.mark.parametrize("over", [None, dict(memory_update_aggregate_write=False, memory_aggregate_momentum_mode="none"),
                                  dict(memory_update_backward_mode="cross_layer_cut")],
                         ids=["aggregated write", "chained writes", "cross_layer_cut"])
def test_two_gpu_ranks_peer_dispatch_combine_matches_data_parallel(tmp_path, over):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), "nccl", str(tmp_path), over), nprocs=2, join=True)
    _check(str(tmp_path), 4e-2, 4e-2, "peer")
