"""Analytic FLOP model and hardware peaks.

``6 * (N - N_emb) + 12 * l * h * q * t`` FLOPs per token (uttt_llm/flame/tools/utils.py:26-38).  Unlike the
reference, the embedding table is found wherever it lives in the module tree, so ``N_emb`` is actually
subtracted.  Fast-weight terms (read ``6*I*D``, write ``12*I*D`` forward, ``30*I*D`` backward per routed row)
are added for the test-time-training models.
"""
from __future__ import annotations

import json
import os
from typing import Tuple

import torch.nn as nn


def get_nparams_and_flops(model: nn.Module, config, seq_len: int) -> Tuple[int, float]:
    n_params = sum(p.numel() for p in model.parameters())
    n_emb = sum(m.weight.numel() for m in model.modules() if isinstance(m, nn.Embedding))
    l, h = config.num_hidden_layers, config.num_heads
    q = config.hidden_size // config.num_heads
    t = min(seq_len, config.window_size) if getattr(config, "window_size", None) else seq_len
    flops = 6 * (n_params - n_emb) + 12 * l * h * q * t
    if getattr(config, "use_memory_block", False):
        rows = config.fw_heads * getattr(config, "memory_num_active_experts", 1)
        per_row = (6 + 12 + 12 + 30) * config.fw_inter_dim * config.fw_head_dim
        flops += l * rows * per_row
    return n_params, float(flops)


def peak_flops() -> float:
    """Dense bf16 peak used for MFU: the measured cuBLAS figure when a ``MEASURED_PEAKS.json`` is present in the
    working directory, else 2.25e15 (B200 nominal)."""
    for cand in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")):
        try:
            with open(cand) as fh:
                return float(json.load(fh)["bf16_tflops"]) * 1e12
        except Exception:
            continue
    return 2.25e15
