"""Per-token-loss (PTL) evaluation: cross-entropy as a function of the position in a long sequence.

* :class:`PerPositionLossTracker` accumulates loss sums / counts per position and reduces them over the
  data-parallel ranks (uttt_llm/flame/utils/per_position_loss_tracker.py:9-177);
* :func:`per_token_loss` computes per-position CE from hidden states with a chunked lm-head so that the
  ``[tokens, vocab]`` logits never exist at once (uttt_llm/flame/eval_loss.py:152-198);
* :func:`evaluate` runs a model over a token source; :func:`summarize` reports the NaN-aware mean over the
  positions at or beyond a cut-off (30000 for 32K rows; uttt_llm/eval/ptl/summarize_ptl.py:26-98).
"""
from __future__ import annotations

import json
import math
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F


class PerPositionLossTracker:
    def __init__(self, seq_len: int, device="cpu"):
        self.loss_sum = torch.zeros(seq_len, dtype=torch.float64, device=device)
        self.count = torch.zeros(seq_len, dtype=torch.float64, device=device)

    def update(self, losses: torch.Tensor, valid: Optional[torch.Tensor] = None) -> None:
        """losses: [b, s] per-token CE; valid: [b, s] bool mask."""
        if valid is None:
            valid = torch.ones_like(losses, dtype=torch.bool)
        s = losses.shape[1]
        self.loss_sum[:s] += (losses.double() * valid).sum(0).to(self.loss_sum.device)
        self.count[:s] += valid.double().sum(0).to(self.count.device)

    def sync_ddp(self, group=None) -> None:
        if dist.is_available() and dist.is_initialized():
            for t in (self.loss_sum, self.count):
                buf = t.cuda() if dist.get_backend(group) == "nccl" and not t.is_cuda else t
                dist.all_reduce(buf, group=group)
                t.copy_(buf)

    def mean(self) -> torch.Tensor:
        return torch.where(self.count > 0, self.loss_sum / self.count.clamp_min(1), torch.full_like(self.count, float("nan")))

    def to_json(self) -> str:
        m = self.mean().tolist()
        return json.dumps({"per_position_loss": [None if math.isnan(x) else x for x in m],
                           "count": self.count.tolist()})


@torch.no_grad()
def per_token_loss(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, chunk: int = 4096) -> torch.Tensor:
    """hidden [b, s, d], weight [V, d], labels [b, s] (already shifted; -100 = ignore) -> [b, s] fp32."""
    b, s, d = hidden.shape
    out = torch.zeros(b * s, device=hidden.device, dtype=torch.float32)
    h, y = hidden.reshape(b * s, d), labels.reshape(-1)
    for i in range(0, b * s, chunk):
        logits = (h[i:i + chunk] @ weight.t().to(h.dtype)).float()
        out[i:i + chunk] = F.cross_entropy(logits, y[i:i + chunk], ignore_index=-100, reduction="none")
    return out.view(b, s)


@torch.no_grad()
def evaluate(model, batches: Iterable[Dict[str, torch.Tensor]], seq_len: int, max_batches: Optional[int] = None,
             device=None) -> PerPositionLossTracker:
    model.eval()
    device = device or next(model.parameters()).device
    tracker = PerPositionLossTracker(seq_len, device)
    for i, batch in enumerate(batches):
        if max_batches is not None and i >= max_batches:
            break
        ids = batch["input_ids"].to(device)
        out = model(input_ids=ids, return_logits=False)
        labels = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], dim=1)
        losses = per_token_loss(out.hidden_states, model.lm_head.weight, labels)
        tracker.update(losses, labels != -100)
    tracker.sync_ddp()
    return tracker


def summarize(per_position: List[Optional[float]], start: int = 30000) -> Dict[str, float]:
    vals = [v for v in per_position[start:] if v is not None and not math.isnan(v)]
    allv = [v for v in per_position if v is not None and not math.isnan(v)]
    return {"ptl_tail_mean": sum(vals) / len(vals) if vals else float("nan"), "tail_positions": len(vals),
            "mean_all": sum(allv) / len(allv) if allv else float("nan"), "start": start}


def main(argv=None):
    """``python -m uttt_b200.eval.ptl --config CFG.json [--checkpoint HF_DIR] [--seq-len 32768] [--batch-size 1]
    [--max-batches 64] [--ptl-start 30000] [--data-files F ...] [--output out.json]``"""
    import argparse
    import json
    from ..config import load_config
    from ..models import build_model
    from ..train.data import build_dataloader
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--checkpoint", default="", help="HF-style folder written by export_hf / dcp-to-hf")
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--max-batches", type=int, default=64)
    ap.add_argument("--ptl-start", type=int, default=30000)
    ap.add_argument("--data-files", nargs="*", default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--output", default="")
    args = ap.parse_args(argv)
    cfg = load_config(args.checkpoint if args.checkpoint else args.config)
    model = build_model(cfg)
    if args.checkpoint:
        import os
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
    loader = build_dataloader("synthetic" if not args.data_files else "files", vocab_size=cfg.vocab_size,
                              seq_len=args.seq_len, batch_size=args.batch_size, rank=0, world=1, seed=0,
                              data_files=args.data_files)
    tracker = evaluate(model, loader, args.seq_len, args.max_batches, torch.device(args.device))
    mean = tracker.mean().tolist()
    per_position = [None if math.isnan(x) else x for x in mean]
    summary = summarize(per_position, min(args.ptl_start, max(args.seq_len - 1, 0)))
    print(json.dumps(summary, sort_keys=True))
    if args.output:
        with open(args.output, "w") as fh:
            fh.write(tracker.to_json())


if __name__ == "__main__":
    main()
