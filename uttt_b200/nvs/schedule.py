"""Chunk schedules of the view-synthesis decoder (uttt_nvs/models/ttt_minimal_v2.py:27-85).

A schedule is a list of ``TTTConfig(start, end, fast_weight, update, apply)`` token ranges: ``apply`` chunks are
decoded with the current fast weights, ``update`` chunks additionally write them afterwards.
"""
from __future__ import annotations

import collections
from typing import List, Optional

TTTConfig = collections.namedtuple("TTTConfig", ["start", "end", "fast_weight", "update", "apply"])


def parallel_ttt_config(update_minibatch: int = 1024, apply_only_minibatch: int = 1024, length: int = 10240,
                        update_length: Optional[int] = None) -> List[TTTConfig]:
    """Alternating (update chunk, apply-only chunk) pairs: posed input view, then the pose-only target view."""
    if update_length is None:
        update_length = length
    assert update_length % (update_minibatch + apply_only_minibatch) == 0
    cfg = []
    for start in range(0, update_length, update_minibatch + apply_only_minibatch):
        cfg.append(TTTConfig(start, start + update_minibatch, True, True, True))
        if apply_only_minibatch > 0:
            cfg.append(TTTConfig(start + update_minibatch, start + update_minibatch + apply_only_minibatch,
                                 False, False, True))
    if update_length < length:
        cfg.append(TTTConfig(update_length, length, False, False, True))
    return cfg


def mini_update_config(update_minibatch: int = 1024, length: int = 10240,
                       update_length: Optional[int] = None) -> List[TTTConfig]:
    if update_length is None:
        update_length = length
    assert update_length % update_minibatch == 0
    cfg = [TTTConfig(s, s + update_minibatch, True, True, False) for s in range(0, update_length, update_minibatch)]
    cfg.append(TTTConfig(0, length, False, False, True))
    return cfg


def compression_ttt_config(minibatch: int = 1024, length: int = 10240) -> List[TTTConfig]:
    return [TTTConfig(s, s + minibatch, True, True, True) for s in range(0, length, minibatch)]


def apply_ttt_config(minibatch: int = 1024, length: int = 10240) -> List[TTTConfig]:
    return [TTTConfig(s, s + minibatch, False, False, True) for s in range(0, length, minibatch)]


def inputs_then_targets_config(num_input: int, num_target: int, tokens_per_view: int) -> List[TTTConfig]:
    """``num_input`` posed views that each read then write, followed by ``num_target`` pose-only views that only
    read (e.g. 4 input + 2 target views)."""
    cfg = [TTTConfig(i * tokens_per_view, (i + 1) * tokens_per_view, True, True, True) for i in range(num_input)]
    base = num_input * tokens_per_view
    cfg += [TTTConfig(base + i * tokens_per_view, base + (i + 1) * tokens_per_view, False, False, True)
            for i in range(num_target)]
    return cfg
