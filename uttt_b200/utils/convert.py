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
