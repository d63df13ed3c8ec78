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
             device=None, chunk: int = 4096) -> PerPositionLossTracker:
    model.eval()
    device = device or next(model.parameters()).device
    tracker = PerPositionLossTracker(seq_len, device)
    for i, batch in enumerate(batches):
        if max_batches is not None and i >= max_batches:
            break
        ids = batch["input_ids"].to(device)
        out = model(input_ids=ids, return_logits=False)
        labels = torch.cat([ids[:, 1:], torch.full_like(ids[:, :1], -100)], dim=1)
        losses = per_token_loss(out.hidden_states, model.lm_head.weight, labels, chunk)
        tracker.update(losses, labels != -100)
    tracker.sync_ddp()
    return tracker


def nan_mean(values) -> float:
    kept = [v for v in values if v is not None and not math.isnan(v)]
    return sum(kept) / len(kept) if kept else math.nan


def load_positions(path) -> List[float]:
    """Per-position mean losses from a result file: the flat JSON list that the evaluation writes
    (``<dump_folder>/<save_prefix>_loss_per_token_position.json``; ``null`` / NaN where nothing was counted), or the
    ``{"per_position_loss": [...], "count": [...]}`` object of ``--output``."""
    with open(path) as fh:
        data = json.load(fh)
    if isinstance(data, dict):
        data = data.get("per_position_loss")
    if not isinstance(data, list) or not data:
        raise ValueError(f"{path}: expected a non-empty JSON list of per-position losses")
    out = []
    for v in data:
        if v is None:
            out.append(math.nan)
        elif isinstance(v, (int, float)) and not isinstance(v, bool):
            out.append(float(v))
        else:
            raise ValueError(f"{path}: non-numeric entry {v!r}")
    return out


def summarize_positions(losses: List[float], min_position: int = 30000, chunks: int = 0) -> Dict[str, object]:
    """The paper's per-token loss: NaN-aware mean over positions >= ``min_position`` (0-based; the last position of
    a row has no next token and is NaN by construction), with the keys of uttt_llm/eval/ptl/summarize_ptl.py:46-64."""
    if min_position < 0 or min_position >= len(losses):
        raise ValueError(f"min_position {min_position} outside 0..{len(losses) - 1}")
    tail = losses[min_position:]
    out: Dict[str, object] = {"positions": len(losses), "min_position": min_position, "tail_positions": len(tail),
                              "tail_nan": sum(1 for v in tail if math.isnan(v)), "ptl": nan_mean(tail),
                              "mean_all": nan_mean(losses)}
    if chunks:
        size = math.ceil(len(losses) / chunks)
        out["chunk_means"] = [nan_mean(losses[i:i + size]) for i in range(0, len(losses), size)][:chunks]
    return out


def summary_main(argv=None) -> int:
    """``python -m uttt_b200.eval.ptl summarize FILE.json [FILE.json ...] [--min-position 30000]
    [--expect-positions 32768] [--chunks N] [--output summaries.json]``  (no GPU, no model)"""
    import argparse
    import sys
    ap = argparse.ArgumentParser(description="Reduce per-position loss files to the per-token-loss number.")
    ap.add_argument("json", nargs="+")
    ap.add_argument("--min-position", type=int, default=30000)
    ap.add_argument("--expect-positions", type=int, default=32768)
    ap.add_argument("--chunks", type=int, default=0)
    ap.add_argument("--output", default=None)
    args = ap.parse_args(argv)
    summaries = {}
    for path in args.json:
        losses = load_positions(path)
        if args.expect_positions and len(losses) != args.expect_positions:
            print(f"warning: {path} has {len(losses)} positions, expected {args.expect_positions}", file=sys.stderr)
        s = summarize_positions(losses, args.min_position, args.chunks)
        summaries[str(path)] = s
        line = f"{path}: PTL(>= {args.min_position}) = {s['ptl']:.4f}  (mean over all positions {s['mean_all']:.4f}"
        if s["tail_nan"]:
            line += f", {s['tail_nan']} NaN position(s) skipped"
        print(line + ")")
        if args.chunks:
            print("  blocks: " + ", ".join(f"{m:.4f}" for m in s["chunk_means"]))
    if args.output:
        with open(args.output, "w") as fh:
            fh.write(json.dumps(summaries, indent=2) + "\n")
    return 0


def job_main(argv) -> int:
    """The reference's job-file interface (uttt_llm/flame/eval_loss.py:905-922, eval/ptl/run.sh):

        torchrun -m uttt_b200.eval.ptl --job.config_file configs/lm/exp/eval_ptl.toml \
            --checkpoint.load_path HF_DIR [--model.config CFG.json] [--training.save_prefix default]
            [--job.dump_folder eval_out] [--eval.lm_head_chunk_size 2048]

    ``training.steps`` batches of ``training.batch_size`` rows of ``training.seq_len`` tokens per rank from
    ``training.data_files``; the ranks' sums are reduced and rank 0 writes
    ``<dump_folder>/<save_prefix>_loss_per_token_position.json`` (a flat list; ``null`` where nothing was counted)."""
    import os
    from ..config import load_config
    from ..config.job_config import JobConfig
    from ..models import build_model
    from ..train.data import build_dataloader
    from ..train.engine import init_distributed
    jc = JobConfig()
    jc.parser.add_argument("--training.save_prefix", type=str, default=None)
    jc.parser.add_argument("--checkpoint.load_path", type=str, default=None)
    jc.parser.add_argument("--eval.per_token_loss_from_hidden", nargs="?", const=True, default=None)
    jc.parser.add_argument("--eval.lm_head_chunk_size", type=int, default=None)
    jc.parse_args(list(argv))
    rank, world, local = init_distributed()
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    ckpt = getattr(jc.checkpoint, "load_path", None)
    model_cfg = getattr(jc.model, "config", None)
    if ckpt and os.path.exists(os.path.join(ckpt, "config.json")):
        cfg = load_config(ckpt)
    elif model_cfg and not str(model_cfg).startswith("PATH/TO/"):
        cfg = load_config(model_cfg)
    else:
        raise SystemExit("give --checkpoint.load_path (a folder with config.json) or --model.config")
    model = build_model(cfg)
    if ckpt:
        st = os.path.join(ckpt, "model.safetensors")
        if os.path.exists(st):
            from safetensors.torch import load_file
            sd = load_file(st)
        else:
            sd = torch.load(os.path.join(ckpt, "pytorch_model.bin"), map_location="cpu")
        model.load_state_dict(sd, strict=False)
    model = model.to(device)
    if device.type == "cuda":
        model = model.bfloat16()
    t = jc.training
    files = getattr(t, "data_files", None)
    if isinstance(files, str):
        if files.startswith("PATH/TO/"):
            raise SystemExit("training.data_files still holds its placeholder value")
        import glob
        files = sorted(glob.glob(files)) or [files]
    loader = build_dataloader("files" if files else "synthetic", vocab_size=cfg.vocab_size, seq_len=int(t.seq_len),
                              batch_size=int(t.batch_size), rank=rank, world=world, seed=int(getattr(t, "seed", 0) or 0),
                              data_files=files)
    tracker = evaluate(model, loader, int(t.seq_len), int(t.steps), device,
                       chunk=int(getattr(getattr(jc, "eval", None), "lm_head_chunk_size", 4096) or 4096))
    if rank == 0:
        out_dir = jc.job.dump_folder
        os.makedirs(out_dir, exist_ok=True)
        prefix = getattr(t, "save_prefix", None) or "default"
        path = os.path.join(out_dir, f"{prefix}_loss_per_token_position.json")
        mean = tracker.mean().tolist()
        with open(path, "w") as fh:
            json.dump([None if math.isnan(x) else x for x in mean], fh)
        print(f"Saved loss at per token to {path}")
        print(f"Number of tokens tracked: {float(tracker.count.sum()) / 1e6}M")
        print(json.dumps(summarize_positions([math.nan if x is None else x for x in load_positions(path)],
                                             min(30000, max(int(t.seq_len) - 1, 0))), sort_keys=True))
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


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
    import sys
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "summarize":
        return summary_main(argv[1:])
    if any(a.startswith("--job.") for a in argv):
        return job_main(argv)
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
