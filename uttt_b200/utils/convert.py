"""Checkpoint converters and corpus preprocessing.

* :func:`dcp_to_hf`: training checkpoint (``step-N`` directory) -> Hugging-Face style directory
  (``config.json`` + ``model.safetensors`` [+ tokenizer files])  (uttt_llm/flame/utils/convert_dcp_to_hf.py:63-118);
* :func:`hf_to_dcp`: the reverse, producing a ``step-0`` seed checkpoint (convert_hf_to_dcp.py:15-26);
* :func:`preprocess`: tokenise text files into arrow shards with an ``input_ids`` column (preprocess.py:12-123).
"""
from __future__ import annotations

import glob
import json
import os
import shutil
from typing import Callable, Iterable, List, Optional

import torch

from ..config import load_config
from ..models import build_model
from ..train.checkpoint import CheckpointManager, export_hf


def dcp_to_hf(checkpoint_dir: str, config_path: str, out_dir: str, tokenizer_path: Optional[str] = None,
              dtype: torch.dtype = torch.float32) -> str:
    cfg = load_config(config_path)
    model = build_model(cfg)
    parent, leaf = os.path.split(os.path.abspath(checkpoint_dir.rstrip("/")))
    mgr = CheckpointManager(os.path.dirname(parent), os.path.basename(parent))
    mgr._load_path(os.path.join(parent, leaf), model, None, None, None, None)
    export_hf(model, cfg, out_dir, dtype)
    if tokenizer_path and os.path.isdir(tokenizer_path):
        for f in glob.glob(os.path.join(tokenizer_path, "token*")) + glob.glob(os.path.join(tokenizer_path, "special*")):
            shutil.copy(f, out_dir)
    return out_dir


def hf_to_dcp(hf_dir: str, dump_folder: str, folder: str = "checkpoint") -> str:
    cfg = load_config(hf_dir)
    model = build_model(cfg)
    st = os.path.join(hf_dir, "model.safetensors")
    if os.path.exists(st):
        from safetensors.torch import load_file
        sd = load_file(st)
    else:
        sd = torch.load(os.path.join(hf_dir, "pytorch_model.bin"), map_location="cpu")
    model.load_state_dict(sd, strict=False)
    mgr = CheckpointManager(dump_folder, folder, interval=1, keep_latest_k=0)
    return mgr.save(0, model, force=True)


def preprocess(files: Iterable[str], out_dir: str, tokenize: Callable[[str], List[int]], shard_docs: int = 1000,
               eos_token_id: Optional[int] = None) -> List[str]:
    """Tokenise one document per line into arrow IPC shards (column ``input_ids``)."""
    import pyarrow as pa
    os.makedirs(out_dir, exist_ok=True)
    shards, docs = [], []

    def flush():
        if not docs:
            return
        path = os.path.join(out_dir, f"data-{len(shards):05d}.arrow")
        table = pa.table({"input_ids": pa.array(docs, type=pa.list_(pa.int32()))})
        with pa.OSFile(path, "wb") as sink, pa.ipc.new_stream(sink, table.schema) as writer:
            writer.write_table(table)
        shards.append(path)
        docs.clear()

    for f in files:
        with open(f, encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                try:
                    line = json.loads(line).get("text", line)
                except (ValueError, AttributeError):
                    pass
                ids = list(tokenize(line))
                if eos_token_id is not None:
                    ids.append(eos_token_id)
                docs.append(ids)
                if len(docs) >= shard_docs:
                    flush()
    flush()
    return shards


def main(argv=None):
    """``python -m uttt_b200.utils.convert dcp-to-hf --checkpoint DIR --config CFG.json --output OUT``
    ``python -m uttt_b200.utils.convert hf-to-dcp --hf-dir DIR --dump-folder RUN``
    ``python -m uttt_b200.utils.convert preprocess --files a.txt b.jsonl --output DIR --tokenizer TOK_DIR``"""
    import argparse
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("dcp-to-hf")
    a.add_argument("--checkpoint", required=True)
    a.add_argument("--config", required=True)
    a.add_argument("--output", required=True)
    a.add_argument("--tokenizer", default=None)
    b = sub.add_parser("hf-to-dcp")
    b.add_argument("--hf-dir", required=True)
    b.add_argument("--dump-folder", required=True)
    c = sub.add_parser("preprocess")
    c.add_argument("--files", nargs="+", required=True)
    c.add_argument("--output", required=True)
    c.add_argument("--tokenizer", default="", help="folder of a HF tokenizer; bytes are used when empty")
    c.add_argument("--shard-docs", type=int, default=1000)
    args = ap.parse_args(argv)
    if args.cmd == "dcp-to-hf":
        print(dcp_to_hf(args.checkpoint, args.config, args.output, args.tokenizer))
    elif args.cmd == "hf-to-dcp":
        print(hf_to_dcp(args.hf_dir, args.dump_folder))
    else:
        if args.tokenizer:
            from transformers import AutoTokenizer
            tok = AutoTokenizer.from_pretrained(args.tokenizer)
            tokenize, eos = (lambda t: tok(t)["input_ids"]), tok.eos_token_id
        else:
            tokenize, eos = (lambda t: list(t.encode("utf-8"))), 0
        print("\n".join(preprocess(args.files, args.output, tokenize, args.shard_docs, eos)))


if __name__ == "__main__":
    main()
