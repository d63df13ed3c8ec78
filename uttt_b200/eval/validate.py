"""Validation loss over a token dataset (the generic evaluation loop: uttt_llm/flame/eval.py:75-743).

    python -m uttt_b200.eval.validate --config CFG.json [--checkpoint HF_DIR] [--seq-len 32768] [--batch-size 1]
        [--max-batches 32] [--data-files F ...] [--device cuda]

Runs the model in eval mode on fixed-length windows and reports the mean next-token loss and perplexity; under
``torch.distributed`` every rank reads its own interleaved windows and the sums are all-reduced.
"""
from __future__ import annotations

import argparse
import json
import math
import os
from typing import Dict, Iterable, Optional

import torch
import torch.distributed as dist


@torch.no_grad()
def validation_loss(model, batches: Iterable[Dict[str, torch.Tensor]], max_batches: Optional[int] = None,
                    device=None) -> Dict[str, float]:
    model.eval()
    device = device or next(model.parameters()).device
    total = torch.zeros(2, dtype=torch.float64, device=device)            # (sum of token losses, tokens)
    for i, batch in enumerate(batches):
        if max_batches is not None and i >= max_batches:
            break
        ids = batch["input_ids"].to(device)
        labels = batch.get("labels", ids).to(device)
        out = model(input_ids=ids, labels=labels)
        n = (labels[:, 1:] != -100).sum()
        total[0] += out.loss.double() * n
        total[1] += n
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(total)
    mean = float(total[0] / total[1].clamp_min(1))
    return {"loss": mean, "perplexity": math.exp(min(mean, 50.0)), "tokens": int(total[1])}


def main(argv=None):
    from ..config import load_config
    from ..models import build_model
    from ..train.data import build_dataloader
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--max-batches", type=int, default=32)
    ap.add_argument("--data-files", nargs="*", default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    cfg = load_config(args.checkpoint if args.checkpoint else args.config)
    model = build_model(cfg)
    if args.checkpoint:
        st = os.path.join(args.checkpoint, "model.safetensors")
        if os.path.exists(st):
            from safetensors.torch import load_file
            sd = load_file(st)
        else:
            sd = torch.load(os.path.join(args.checkpoint, "pytorch_model.bin"), map_location="cpu")
        model.load_state_dict(sd, strict=False)
    model = model.to(args.device)
    if args.device.startswith("cuda"):
        model = model.bfloat16()
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    loader = build_dataloader("synthetic" if not args.data_files else "files", vocab_size=cfg.vocab_size,
                              seq_len=args.seq_len, batch_size=args.batch_size, rank=rank, world=world, seed=0,
                              data_files=args.data_files)
    print(json.dumps(validation_loss(model, loader, args.max_batches, torch.device(args.device)), sort_keys=True))


if __name__ == "__main__":
    main()
