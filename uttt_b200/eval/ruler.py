"""Long-context retrieval evaluation in the style of RULER's needle-in-a-haystack tasks.

The reference drives the ``lm_eval`` harness (uttt_llm/eval/ruler/run_ruler_eval.py:28-363); that package is
not available offline, so the tasks are generated here directly on token ids: a haystack of filler tokens
with ``key -> value`` needles inserted at controlled depths, a query for one key at the end, and exact match
of the greedily decoded value.  Samples can be sharded over ranks / jobs and the shard results merged
(merge_ruler_shards.py).
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import torch

from ..models.generation import generate


def make_niah_sample(vocab_size: int, length: int, num_needles: int, value_len: int, seed: int,
                     reserved: int = 16) -> Dict[str, torch.Tensor]:
    """Returns {'prompt': [length] ids, 'answer': [value_len] ids}.  Token ids below ``reserved`` are markers:
    1 = needle start, 2 = needle separator, 3 = query marker."""
    g = torch.Generator().manual_seed(seed)
    hay = torch.randint(reserved, vocab_size, (length,), generator=g)
    keys = torch.randint(reserved, vocab_size, (num_needles,), generator=g)
    vals = torch.randint(reserved, vocab_size, (num_needles, value_len), generator=g)
    span = value_len + 3
    usable = length - (span + 2) - 1
    depths = torch.linspace(0.05, 0.95, num_needles)
    for i in range(num_needles):
        pos = int(depths[i] * usable)
        hay[pos] = 1
        hay[pos + 1] = keys[i]
        hay[pos + 2] = 2
        hay[pos + 3:pos + 3 + value_len] = vals[i]
    target = int(torch.randint(0, num_needles, (1,), generator=g))
    hay[-3], hay[-2], hay[-1] = 3, keys[target], 2
    return {"prompt": hay, "answer": vals[target]}


@torch.no_grad()
def run_niah(model, vocab_size: int, length: int, num_samples: int = 8, num_needles: int = 4, value_len: int = 4,
             shard: int = 0, num_shards: int = 1, device=None) -> Dict[str, float]:
    device = device or next(model.parameters()).device
    hits, total = 0, 0
    for idx in range(shard, num_samples, num_shards):
        s = make_niah_sample(vocab_size, length, num_needles, value_len, seed=idx)
        out = generate(model, s["prompt"][None].to(device), max_new_tokens=value_len)
        hits += int(torch.equal(out[0, -value_len:].cpu(), s["answer"]))
        total += 1
    return {"task": "niah", "length": length, "shard": shard, "num_shards": num_shards, "hits": hits, "total": total,
            "accuracy": hits / max(total, 1)}


def merge_shards(results: List[Dict[str, float]]) -> Dict[str, float]:
    hits, total = sum(r["hits"] for r in results), sum(r["total"] for r in results)
    return {"task": results[0]["task"], "length": results[0]["length"], "hits": hits, "total": total,
            "accuracy": hits / max(total, 1), "shards": len(results)}


def main(argv=None):
    """``python -m uttt_b200.eval.ruler --config CFG.json [--checkpoint HF_DIR] [--length 4096] [--num-samples 8]
    [--shard I --num-shards S] [--output shard.json]`` or ``--merge a.json b.json ...``"""
    import argparse
    import json
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="")
    ap.add_argument("--checkpoint", default="")
    ap.add_argument("--length", type=int, default=4096)
    ap.add_argument("--num-samples", type=int, default=8)
    ap.add_argument("--num-needles", type=int, default=4)
    ap.add_argument("--value-len", type=int, default=4)
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--num-shards", type=int, default=1)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--output", default="")
    ap.add_argument("--merge", nargs="*", default=None, help="merge shard result files instead of running")
    args = ap.parse_args(argv)
    if args.merge:
        results = [json.load(open(f)) for f in args.merge]
        print(json.dumps(merge_shards(results), sort_keys=True))
        return
    from ..config import load_config
    from ..models import build_model
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
    model = model.to(args.device).eval()
    res = run_niah(model, cfg.vocab_size, args.length, args.num_samples, args.num_needles, args.value_len, args.shard,
                   args.num_shards, torch.device(args.device))
    print(json.dumps(res, sort_keys=True))
    if args.output:
        with open(args.output, "w") as fh:
            json.dump(res, fh)


if __name__ == "__main__":
    main()
