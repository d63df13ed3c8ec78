"""RULER through the ``lm_eval`` harness, for the language models of this package.

The reference evaluates long-context retrieval by handing an HF checkpoint folder to
``lm_eval.evaluator.simple_evaluate`` with strided sample shards, and merges the shard results afterwards
(uttt_llm/eval/ruler/run_ruler_eval.py:28-363, merge_ruler_shards.py).  Here the model is not an HF class, so
the harness gets an adapter instead:

* :class:`TextAdapter` implements the three request kinds of the harness (``generate_until``, ``loglikelihood``,
  ``loglikelihood_rolling``) on a model of this package and a tokenizer with ``encode`` / ``decode``.  It needs
  neither ``lm_eval`` nor ``transformers`` and is what the tests drive.
* :func:`as_harness_model` wraps an adapter in a subclass of ``lm_eval.api.model.LM`` (imported when called).
* ``python -m uttt_b200.eval.harness --model-dir HF_DIR --output results.json [--tasks ruler] [--max-length 32768]
  [--limit N] [--sample-shard-rank r --sample-shard-world-size w] [--seed S] [--log-samples]`` takes the reference's
  flags and writes the same files: ``results.json``, ``sample_shard_manifest.json`` and, with ``--log-samples``,
  ``samples/<task>.jsonl``.  ``merge --shards-dir D --output-dir O --expected-shards N`` pools the per-task scores of
  the shards weighted by their sample counts.

Without ``lm_eval`` the command stops with a message that names ``python -m uttt_b200.eval.ruler``, the self-contained
needle tasks that need no external package.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch


def _args_of(request) -> tuple:
    return tuple(request.args) if hasattr(request, "args") else tuple(request)


def first_stop(text: str, stops: Sequence[str]) -> str:
    """``text`` cut before the earliest stop string that occurs in it."""
    cut = len(text)
    for s in stops:
        if s:
            i = text.find(s)
            if i >= 0:
                cut = min(cut, i)
    return text[:cut]


def strided_samples(totals: Dict[str, int], rank: int, world: int) -> Tuple[Optional[Dict[str, List[int]]], dict]:
    """Sample indices ``rank, rank + world, ...`` per task and the manifest the reference writes beside the results
    (run_ruler_eval.py:198-249)."""
    if world <= 1:
        return None, {"enabled": False, "rank": rank, "world_size": world, "tasks": {}}
    if not 0 <= rank < world:
        raise ValueError(f"sample shard rank must be in [0, {world}), got {rank}")
    samples, manifest = {}, {}
    for task, total in totals.items():
        idx = list(range(rank, total, world))
        if idx:
            samples[task] = idx
            manifest[task] = {"total_samples": total, "shard_samples": len(idx), "first_index": idx[0],
                              "last_index": idx[-1]}
    if not samples:
        raise ValueError(f"sample shard rank {rank}/{world} received no samples")
    return samples, {"enabled": True, "rank": rank, "world_size": world, "tasks": manifest}


class TextAdapter:
    """Harness requests on a causal LM of this package.  ``tokenizer`` needs ``encode(str) -> ids`` and
    ``decode(ids) -> str``; batch size is one request (the chunk-recurrent cache takes no padding)."""

    def __init__(self, model, tokenizer, max_length: int = 32768, device=None, max_gen_toks: int = 256,
                 eos_token_id: Optional[int] = None):
        self.model = model.eval()
        self.tokenizer = tokenizer
        self.max_length = int(max_length)
        self.max_gen_toks = int(max_gen_toks)
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.eos_token_id = eos_token_id if eos_token_id is not None else getattr(tokenizer, "eos_token_id", None)

    # tokenizer ---------------------------------------------------------------------------------------------------
    def encode(self, text: str) -> List[int]:
        try:
            return list(self.tokenizer.encode(text, add_special_tokens=False))
        except TypeError:
            return list(self.tokenizer.encode(text))

    def decode(self, ids: Iterable[int]) -> str:
        return self.tokenizer.decode(list(ids))

    # requests ----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_until(self, requests) -> List[str]:
        results = []
        for req in requests:
            context, kwargs = _args_of(req)
            kwargs = dict(kwargs or {})
            until = kwargs.get("until") or []
            until = [until] if isinstance(until, str) else list(until)
            budget = int(kwargs.get("max_gen_toks", self.max_gen_toks))
            ids = self.encode(context)[-max(self.max_length - budget, 1):]          # keep the end of the prompt
            tokens = torch.tensor([ids], dtype=torch.long, device=self.device)
            out = self.model(input_ids=tokens, use_cache=True, logits_to_keep=1)
            new: List[int] = []
            text = ""
            for _ in range(budget):
                nxt = int(out.logits[0, -1].float().argmax())
                if self.eos_token_id is not None and nxt == self.eos_token_id:
                    break
                new.append(nxt)
                text = self.decode(new)
                if any(s and s in text for s in until):
                    break
                out = self.model(input_ids=torch.tensor([[nxt]], device=self.device),
                                 past_key_values=out.past_key_values, use_cache=True, logits_to_keep=1)
            results.append(first_stop(text, until))
        return results

    @torch.no_grad()
    def _score(self, context_ids: List[int], continuation_ids: List[int]) -> Tuple[float, bool]:
        ids = (context_ids + continuation_ids)[-(self.max_length + 1):]
        n = min(len(continuation_ids), len(ids) - 1)
        tokens = torch.tensor([ids[:-1]], dtype=torch.long, device=self.device)
        logits = self.model(input_ids=tokens, use_cache=False, logits_to_keep=n).logits[0].float()
        target = torch.tensor(ids[-n:], device=self.device)
        logp = torch.log_softmax(logits, dim=-1)
        picked = logp.gather(1, target[:, None])[:, 0]
        return float(picked.sum()), bool((logp.argmax(-1) == target).all())

    def loglikelihood(self, requests) -> List[Tuple[float, bool]]:
        out = []
        for req in requests:
            context, continuation = _args_of(req)[:2]
            ctx = self.encode(context) if context else []
            if not ctx:                                          # the harness scores from the end-of-text token
                ctx = [self.eos_token_id if self.eos_token_id is not None else 0]
            out.append(self._score(ctx, self.encode(continuation)))
        return out

    def loglikelihood_rolling(self, requests) -> List[float]:
        out = []
        for req in requests:
            ids = self.encode(_args_of(req)[0])
            prefix = [self.eos_token_id if self.eos_token_id is not None else 0]
            total = 0.0
            for start in range(0, len(ids), self.max_length):                       # disjoint windows
                window = ids[start:start + self.max_length]
                total += self._score(prefix, window)[0]
                prefix = [window[-1]]
            out.append(total)
        return out


def as_harness_model(adapter: TextAdapter):
    """An ``lm_eval.api.model.LM`` that forwards to ``adapter``."""
    from lm_eval.api.model import LM

    class _Harness(LM):
        def __init__(self):
            super().__init__()
            self.adapter = adapter

        def generate_until(self, requests, disable_tqdm: bool = False):
            return adapter.generate_until(requests)

        def loglikelihood(self, requests, disable_tqdm: bool = False):
            return adapter.loglikelihood(requests)

        def loglikelihood_rolling(self, requests, disable_tqdm: bool = False):
            return adapter.loglikelihood_rolling(requests)

        @property
        def tokenizer_name(self) -> str:
            return getattr(adapter.tokenizer, "name_or_path", "tokenizer")

    return _Harness()


def load_model_dir(model_dir: str, device: str, dtype: str = "bfloat16"):
    """Model and tokenizer of an HF-style folder (``config.json`` + weights + tokenizer files)."""
    from ..config import load_config
    from ..models import build_model
    cfg = load_config(model_dir)
    model = build_model(cfg)
    st = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file
        sd = load_file(st)
    else:
        sd = torch.load(os.path.join(model_dir, "pytorch_model.bin"), map_location="cpu", weights_only=True)
    model.load_state_dict(sd, strict=True)
    torch_dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[dtype]
    model = model.to(device=device, dtype=torch_dtype if str(device).startswith("cuda") else torch.float32)
    from transformers import AutoTokenizer
    return model, AutoTokenizer.from_pretrained(model_dir)


def write_samples(samples, output_dir: Path) -> List[str]:
    if not samples:
        return []
    folder = output_dir / "samples"
    folder.mkdir(parents=True, exist_ok=True)
    written = []
    for task, records in (samples.items() if isinstance(samples, dict) else [("samples", samples)]):
        path = folder / (re.sub(r"[^A-Za-z0-9_.-]+", "_", str(task)).strip("_") or "samples")
        path = path.with_name(path.name + ".jsonl")
        with open(path, "w", encoding="utf-8") as fh:
            for rec in records if isinstance(records, list) else [records]:
                fh.write(json.dumps(rec, sort_keys=True, default=str) + "\n")
        written.append(str(path.relative_to(output_dir)))
    return written


def merge_results(shards: Sequence[dict]) -> dict:
    """Per-task metrics pooled over shards, each shard weighted by its number of samples of that task."""
    merged: Dict[str, Dict[str, float]] = {}
    weights: Dict[str, float] = {}
    for doc in shards:
        counts = doc.get("sample_shard", {}).get("tasks", {})
        for task, metrics in doc.get("results", {}).items():
            w = float(counts.get(task, {}).get("shard_samples", doc.get("n-samples", {}).get(task, {})
                                               .get("effective", 1)))
            weights[task] = weights.get(task, 0.0) + w
            slot = merged.setdefault(task, {})
            for name, value in metrics.items():
                if isinstance(value, (int, float)) and not isinstance(value, bool) and "stderr" not in name:
                    slot[name] = slot.get(name, 0.0) + w * float(value)
    return {"results": {t: {k: v / weights[t] for k, v in m.items()} for t, m in merged.items()},
            "samples_per_task": weights, "shards": len(shards)}


def _merge_main(argv) -> int:
    ap = argparse.ArgumentParser(prog="harness merge")
    ap.add_argument("--shards-dir", type=Path, required=True)
    ap.add_argument("--output-dir", type=Path, required=True)
    ap.add_argument("--expected-shards", type=int, required=True)
    args = ap.parse_args(argv)
    files = sorted(args.shards_dir.glob("*/results.json"))
    if len(files) != args.expected_shards:
        print(f"expected {args.expected_shards} shard results under {args.shards_dir}, found {len(files)}",
              file=sys.stderr)
        return 1
    docs = [json.loads(f.read_text()) for f in files]
    ranks = sorted(d.get("sample_shard", {}).get("rank", -1) for d in docs)
    if ranks != list(range(args.expected_shards)):
        print(f"shard ranks {ranks} are not 0..{args.expected_shards - 1}", file=sys.stderr)
        return 1
    args.output_dir.mkdir(parents=True, exist_ok=True)
    out = args.output_dir / "results.json"
    out.write_text(json.dumps(merge_results(docs), indent=2, sort_keys=True) + "\n")
    print(out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "merge":
        return _merge_main(argv[1:])
    ap = argparse.ArgumentParser(description="RULER (or any harness task) on a model folder of this package.")
    ap.add_argument("--model-dir", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--max-length", type=int, default=32768)
    ap.add_argument("--tasks", default="ruler")
    ap.add_argument("--batch-size", default="1")
    ap.add_argument("--limit", type=float, default=None)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--log-samples", action="store_true")
    ap.add_argument("--metadata-max-lengths", default="4096,8192,16384,32768")
    ap.add_argument("--sample-shard-rank", type=int, default=0)
    ap.add_argument("--sample-shard-world-size", type=int, default=1)
    args = ap.parse_args(argv)
    try:
        from lm_eval import evaluator
        from lm_eval.tasks import TaskManager
    except ImportError:
        print("the lm_eval package is not installed; `python -m uttt_b200.eval.ruler` runs the self-contained needle "
              "tasks without it", file=sys.stderr)
        return 2
    if args.seed is not None:
        torch.manual_seed(args.seed)
    model, tokenizer = load_model_dir(args.model_dir, args.device, args.dtype)
    adapter = TextAdapter(model, tokenizer, args.max_length, args.device)
    lengths = [int(v) for v in args.metadata_max_lengths.split(",") if v.strip()] or [args.max_length]
    metadata = {"max_seq_lengths": lengths, "pretrained": str(args.model_dir), "tokenizer": str(args.model_dir),
                "max_length": args.max_length}
    tasks = [t.strip() for t in args.tasks.split(",") if t.strip()]
    samples, manifest = None, {"enabled": False, "rank": args.sample_shard_rank,
                               "world_size": args.sample_shard_world_size, "tasks": {}}
    if args.sample_shard_world_size > 1:
        loaded = TaskManager(metadata=metadata).load(tasks)
        totals = {name: len(task.eval_docs) for name, task in loaded["tasks"].items()}
        samples, manifest = strided_samples(totals, args.sample_shard_rank, args.sample_shard_world_size)
    results = evaluator.simple_evaluate(model=as_harness_model(adapter), tasks=tasks, batch_size=args.batch_size,
                                        limit=args.limit, samples=samples, bootstrap_iters=0,
                                        log_samples=args.log_samples, metadata=metadata)
    if results is None:
        return 0
    out = Path(args.output).resolve()
    out.parent.mkdir(parents=True, exist_ok=True)
    files = write_samples(results.pop("samples", None), out.parent)
    if files:
        results["sample_files"] = files
    results["sample_shard"] = manifest
    (out.parent / "sample_shard_manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    out.write_text(json.dumps(results, indent=2, sort_keys=True, default=str) + "\n")
    print(out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
