"""Token data sources for the language-model trainer.

* :class:`SyntheticZipfTokens` - deterministic Zipf(s)-distributed token ids of a fixed
  sequence length (benchmarks and tests; there is no dataset on the benchmark machines).
* :class:`PackedTokenDataset` - fixed-length packing of a tokenised corpus (``.npy`` / ``.bin``
  uint16/int32 token streams, or arrow/parquet files with an ``input_ids`` / ``text`` column),
  sharded by data-parallel rank; the counterpart of ``OnlineTokenizedIterableDataset`` +
  ``ParallelAwareDataLoader`` (uttt_llm/flame/data.py:179-246, 537-578).

Both are resumable: ``state_dict()`` / ``load_state_dict()`` capture the position, and batches
are produced in pinned host memory so the trainer can overlap the host-to-device copy.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch


def zipf_probs(vocab: int, s: float = 1.1) -> np.ndarray:
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    p = ranks ** (-s)
    return p / p.sum()


class SyntheticZipfTokens:
    """Infinite stream of [batch, seq_len] int64 token ids ~ Zipf(s) over the vocabulary."""

    def __init__(self, vocab_size: int, seq_len: int, batch_size: int, seed: int = 0, s: float = 1.1,
                 rank: int = 0, world: int = 1, pin: bool = True):
        self.vocab_size, self.seq_len, self.batch_size = vocab_size, seq_len, batch_size
        self.seed, self.rank, self.world = seed, rank, world
        self.cdf = np.cumsum(zipf_probs(vocab_size, s))
        self.cdf[-1] = 1.0
        self.step = 0
        self.pin = pin and torch.cuda.is_available()

    def _batch(self, step: int) -> torch.Tensor:
        rng = np.random.default_rng([self.seed, self.rank, step])
        u = rng.random((self.batch_size, self.seq_len))
        ids = np.searchsorted(self.cdf, u, side="right").astype(np.int64)
        t = torch.from_numpy(np.minimum(ids, self.vocab_size - 1))
        return t.pin_memory() if self.pin else t

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        ids = self._batch(self.step)
        self.step += 1
        return {"input_ids": ids, "labels": ids}

    def state_dict(self) -> Dict[str, int]:
        return {"step": self.step}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.step = int(sd["step"])


def _load_token_file(path: str) -> np.ndarray:
    if path.endswith(".npy"):
        return np.load(path, mmap_mode="r")
    if path.endswith(".bin"):
        return np.memmap(path, dtype=np.uint16, mode="r")
    if path.endswith((".arrow", ".parquet")):
        import pyarrow as pa
        import pyarrow.parquet as pq
        if path.endswith(".parquet"):
            table = pq.read_table(path)
        else:
            try:
                table = pa.ipc.open_stream(path).read_all()
            except pa.ArrowInvalid:
                table = pa.ipc.open_file(path).read_all()
        if "input_ids" not in table.column_names:
            raise ValueError(f"{path}: expected a tokenised `input_ids` column (run the preprocess tool first)")
        return np.concatenate([np.asarray(x, dtype=np.int64) for x in table.column("input_ids").to_pylist()])
    raise ValueError(f"unsupported token file {path}")


class PackedTokenDataset:
    """Concatenate token streams and cut fixed ``seq_len`` windows; rank r takes windows r, r+world, ..."""

    def __init__(self, files: str | List[str], seq_len: int, batch_size: int, rank: int = 0, world: int = 1,
                 seed: int = 0, shuffle: bool = True, pin: bool = True):
        paths = sorted(glob.glob(files)) if isinstance(files, str) else list(files)
        if not paths:
            raise FileNotFoundError(f"no data files match {files!r}")
        self.streams = [_load_token_file(p) for p in paths]
        self.seq_len, self.batch_size, self.rank, self.world = seq_len, batch_size, rank, world
        self.seed, self.shuffle = seed, shuffle
        self.windows = [(si, off) for si, s in enumerate(self.streams)
                        for off in range(0, len(s) - seq_len + 1, seq_len)]
        if len(self.windows) < world * batch_size:
            raise ValueError("dataset too small for one global batch")
        self.epoch, self.cursor = 0, 0
        self.pin = pin and torch.cuda.is_available()

    def _order(self, epoch: int) -> np.ndarray:
        idx = np.arange(len(self.windows))
        if self.shuffle:
            np.random.default_rng([self.seed, epoch]).shuffle(idx)
        return idx[self.rank::self.world]

    def __iter__(self):
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        order = self._order(self.epoch)
        if self.cursor + self.batch_size > len(order):
            self.epoch, self.cursor = self.epoch + 1, 0
            order = self._order(self.epoch)
        rows = []
        for w in order[self.cursor:self.cursor + self.batch_size]:
            si, off = self.windows[int(w)]
            rows.append(np.asarray(self.streams[si][off:off + self.seq_len], dtype=np.int64))
        self.cursor += self.batch_size
        ids = torch.from_numpy(np.stack(rows))
        ids = ids.pin_memory() if self.pin else ids
        return {"input_ids": ids, "labels": ids}

    def state_dict(self) -> Dict[str, int]:
        return {"epoch": self.epoch, "cursor": self.cursor}

    def load_state_dict(self, sd: Dict[str, int]) -> None:
        self.epoch, self.cursor = int(sd["epoch"]), int(sd["cursor"])


def build_dataloader(dataset: str, *, vocab_size: int, seq_len: int, batch_size: int, rank: int, world: int,
                     seed: int = 0, data_files: Optional[str] = None, **text_options):
    """``synthetic``: Zipf ids; ``tokens``: pre-tokenised ``.npy`` / ``.bin`` / arrow / parquet streams packed in
    process; anything else (``arrow``, ``parquet``, ``json``, ``text``, a dataset path, comma-separated lists):
    the text pipeline of :mod:`uttt_b200.train.text_data` (online tokenisation, packing, workers, interleave)."""
    if dataset in ("synthetic", "zipf"):
        return SyntheticZipfTokens(vocab_size, seq_len, batch_size, seed=seed, rank=rank, world=world)
    if dataset in ("tokens", "packed") or (data_files or "").endswith((".npy", ".bin")):
        return PackedTokenDataset(data_files, seq_len, batch_size, rank=rank, world=world, seed=seed)
    from .text_data import build_text_dataloader
    return build_text_dataloader(dataset, seq_len=seq_len, batch_size=batch_size, rank=rank, world=world, seed=seed,
                                 data_files=data_files, **text_options)
