"""The view-synthesis trainer on two gloo ranks: training, the in-training evaluation (per-rank batches, averaged
metrics), visuals and the checkpoint written by rank 0 from the gathered optimizer state, then a resume."""
import json
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


def _worker(rank: int, world: int, port: int, folder: str):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    os.environ.pop("UTTT_NVS_OUT_DIR", None)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from test_nvs_cpu import _cfg
    from uttt_b200.nvs.trainer import NVSTrainer
    cfg = _cfg()
    cfg["training"].update(out_dir=folder, batch_size_per_gpu=1, total_batch_size=2, max_fwdbwd_passes=4, eval_every=2,
                           vis_every=4, eval_num_views=5, checkpoint_every=4, print_every=100)
    t = NVSTrainer(cfg, device=torch.device("cpu"))
    first = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    t.fit()
    weights = torch.cat([p.detach().flatten().float() for p in t.model.parameters()])
    t2 = NVSTrainer(cfg, device=torch.device("cpu"))
    resumed = torch.cat([p.detach().flatten().float() for p in t2.model.parameters()])
    torch.save({"weights": weights, "resumed": resumed, "step": t2.fwdbwd_step, "updates": t2.update_step,
                "moved": bool(any((p.detach() - first[n]).abs().max() > 0 for n, p in t.model.named_parameters()))},
               os.path.join(folder, f"result.{rank}"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_train_evaluate_save_and_resume(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = (torch.load(tmp_path / f"result.{r}") for r in range(2))
    assert a["moved"] and torch.equal(a["weights"], b["weights"])            # the ranks stay in step
    assert a["step"] == b["step"] == 4 and a["updates"] == 4
    torch.testing.assert_close(a["resumed"], a["weights"], atol=1e-2, rtol=1e-2)    # fp32 masters -> compute copies
    run = tmp_path / "t"
    made = set(os.listdir(run))
    assert {"ckpt_0000000000000004.pt", "eval_00000001", "eval_00000002", "eval_00000004", "iter_00000004",
            "metrics.jsonl"} <= made
    lines = [json.loads(ln) for ln in open(run / "metrics.jsonl")]
    assert [ln["step"] for ln in lines if "eval/loss" in ln] == [1, 2, 4]
    assert len([ln for ln in lines if "train/loss" in ln]) == 4              # written once, by rank 0
