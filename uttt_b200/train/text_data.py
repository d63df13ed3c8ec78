"""Text data pipeline of the language-model trainer: documents -> online tokenisation -> fixed-length packing.

Counterpart of the reference's ``OnlineTokenizedIterableDataset`` / ``DataCollatorForLanguageModeling`` /
``ParallelAwareDataLoader`` / ``build_dataset`` (uttt_llm/flame/data.py:179-246, 347-534, 537-578, 581-763), written
around an explicit, picklable cursor instead of nested iterator states:

* a *source* is any HF ``datasets`` dataset (arrow / parquet / json / text files, streaming or map-style) or a plain
  list of samples; rank ``r`` of ``W`` data-parallel ranks with ``N`` loader workers reads samples
  ``i % (W * N) == r * N + worker``;
* samples carry ``text`` / ``content`` (tokenised on the fly, 64 documents per tokenizer call) or ``input_ids``
  (kept as they are, so pre-tokenised evaluation rows keep their exact length);
* tokens are appended to a buffer and cut into ``seq_len`` windows; the state (samples consumed + left-over tokens)
  restores the stream exactly;
* several sources are interleaved sample by sample with probabilities ``data_probs`` from a seeded generator;
* the collator stacks (and pads, masking the labels) or, with ``varlen``, emits one concatenated row with
  ``cu_seqlens`` cut at BOS (or after EOS) and at ``context_len``.
"""
from __future__ import annotations

import copy
import os
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------- tokenizers
class ByteTokenizer:
    """UTF-8 bytes + BOS / EOS / PAD (vocabulary 259).  Stands in where no tokenizer files are available
    (``--model.tokenizer_path byte``); real runs pass a local ``transformers`` tokenizer directory."""

    bos_token_id, eos_token_id, pad_token_id = 256, 257, 258
    vocab_size = 259

    def __call__(self, texts, return_attention_mask: bool = False, **_) -> Dict[str, List[List[int]]]:
        if isinstance(texts, str):
            texts = [texts]
        return {"input_ids": [[self.bos_token_id] + list(t.encode("utf-8")) + [self.eos_token_id] for t in texts]}

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


def load_tokenizer(path: Optional[str]):
    if not path or path == "byte":
        return ByteTokenizer()
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(path, trust_remote_code=False)


# ----------------------------------------------------------------------------- sources
def load_text_source(dataset: str, dataset_name: Optional[str] = None, dataset_split: str = "train",
                     data_dir: Optional[str] = None, data_files: Optional[str] = None, streaming: bool = False,
                     seed: Optional[int] = None):
    """One HF ``datasets`` dataset.  ``dataset`` is a builder name ('arrow', 'parquet', 'json', 'text', 'csv') with
    ``data_files`` / ``data_dir``, or a dataset path.  Map-style datasets are shuffled with ``seed`` (their order is
    recoverable); streaming ones use the library's buffer shuffle."""
    from datasets import load_dataset
    ds = load_dataset(path=dataset, name=dataset_name, split=dataset_split, data_dir=data_dir, data_files=data_files,
                      streaming=streaming)
    if seed is not None:
        ds = ds.shuffle(seed=seed) if not streaming else ds.shuffle(seed=seed, buffer_size=1024)
    return ds


class _ListSource:
    """A list of samples with the two methods the packer needs (tests, tiny corpora)."""

    def __init__(self, samples: Sequence[Dict[str, Any]]):
        self.samples = list(samples)

    def __iter__(self):
        return iter(self.samples)


def _strided(source: Iterable[Dict[str, Any]], index: int, stride: int, skip: int) -> Iterator[Dict[str, Any]]:
    """Samples ``index, index + stride, ...`` of ``source``, resuming after ``skip`` of them."""
    if hasattr(source, "shard") and hasattr(source, "num_shards") and getattr(source, "num_shards", 0) >= stride \
            and source.num_shards % stride == 0:
        it = iter(source.shard(num_shards=stride, index=index))      # file-level sharding: no wasted reads
        for n, sample in enumerate(it):
            if n >= skip:
                yield sample
        return
    taken = 0
    for n, sample in enumerate(source):
        if n % stride != index:
            continue
        if taken >= skip:
            yield sample
        taken += 1


class InterleavedSources:
    """Sample-by-sample mixture of several sources with probabilities ``probs`` (seeded; exhausted sources restart,
    as an infinite training stream needs).  ``skip`` replays the same choices without reading the skipped samples
    twice from the sources that support cheap skipping."""

    def __init__(self, sources: Sequence[Iterable[Dict[str, Any]]], probs: Optional[Sequence[float]] = None,
                 seed: int = 0):
        self.sources = list(sources)
        p = np.asarray(probs if probs is not None else [1.0] * len(self.sources), dtype=np.float64)
        if len(p) != len(self.sources) or (p < 0).any() or p.sum() <= 0:
            raise ValueError("data_probs needs one non-negative weight per dataset")
        self.probs = p / p.sum()
        self.seed = seed

    def __iter__(self):
        rng = np.random.default_rng(self.seed)
        its = [iter(s) for s in self.sources]
        while True:
            i = int(rng.choice(len(its), p=self.probs))
            try:
                yield next(its[i])
            except StopIteration:
                its[i] = iter(self.sources[i])
                yield next(its[i])


# ----------------------------------------------------------------------------- tokenise + pack
class OnlineTokenizedPacker:
    """Infinite iterator of ``{'input_ids': LongTensor[seq_len]}`` for one (rank, worker) slice of a source."""

    TOKENIZE_BATCH = 64

    def __init__(self, source, tokenizer, seq_len: int, rank: int = 0, world: int = 1, worker: int = 0,
                 workers: int = 1):
        self.source, self.tokenizer, self.seq_len = source, tokenizer, int(seq_len)
        self.index, self.stride = rank * max(workers, 1) + worker, world * max(workers, 1)
        self.consumed = 0                 # samples of this slice whose tokens are entirely in `tokens` or emitted
        self.epoch = 0
        self.tokens: List[int] = []

    def _documents(self) -> Iterator[List[int]]:
        """Token lists of the slice's documents in order, from the cursor on; text is tokenised in batches."""
        pending: List[str] = []

        def flush():
            if pending:
                for ids in self.tokenizer(list(pending), return_attention_mask=False)["input_ids"]:
                    yield list(ids)
                pending.clear()
        while True:
            seen = 0
            for sample in _strided(self.source, self.index, self.stride, self.consumed):
                seen += 1
                if sample.get("input_ids") is not None:
                    yield from flush()
                    yield list(sample["input_ids"])
                    continue
                text = sample.get("text", sample.get("content"))
                if text is None:
                    raise ValueError(f"sample has neither 'text', 'content' nor 'input_ids': {list(sample)}")
                pending.append(text)
                if len(pending) == self.TOKENIZE_BATCH:
                    yield from flush()
            yield from flush()
            if seen == 0 and self.consumed == 0:
                raise ValueError("the data source yields no samples for this rank")
            self.epoch += 1                # the slice is exhausted: start over (an epoch boundary of the stream)
            self.consumed = 0

    def __iter__(self):
        for ids in self._documents():
            self.tokens.extend(ids)
            self.consumed += 1
            while len(self.tokens) >= self.seq_len:
                window = torch.tensor(self.tokens[:self.seq_len], dtype=torch.long)
                del self.tokens[:self.seq_len]
                yield {"input_ids": window}

    def state_dict(self) -> Dict[str, Any]:
        return {"consumed": self.consumed, "epoch": self.epoch, "tokens": copy.copy(self.tokens)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.consumed, self.epoch, self.tokens = int(sd["consumed"]), int(sd.get("epoch", 0)), list(sd["tokens"])


# ----------------------------------------------------------------------------- collator
class LMCollator:
    """``varlen=False``: ``input_ids`` / ``labels`` [B, S] (+ ``attention_mask``; rows of different lengths are padded
    with the pad id and their labels masked with -100).  ``varlen=True``: the rows are concatenated into ONE row
    [1, total] with ``cu_seqlens`` [n + 1] int32: document starts at BOS tokens (or after EOS tokens when the
    tokenizer has no BOS), and no span longer than ``context_len``."""

    def __init__(self, tokenizer, context_len: Optional[int] = None, varlen: bool = False):
        self.tokenizer, self.context_len, self.varlen = tokenizer, context_len, varlen

    def __call__(self, examples: List[Any]) -> Dict[str, torch.Tensor]:
        rows = [torch.as_tensor(e["input_ids"] if isinstance(e, dict) else e, dtype=torch.long) for e in examples]
        if not self.varlen:
            longest = max(int(r.numel()) for r in rows)
            if all(int(r.numel()) == longest for r in rows):
                ids = torch.stack(rows)
                mask = torch.ones_like(ids)
            else:
                pad = getattr(self.tokenizer, "pad_token_id", None)
                if pad is None:
                    raise ValueError("rows of different lengths need a tokenizer with a pad token")
                ids = torch.full((len(rows), longest), int(pad), dtype=torch.long)
                mask = torch.zeros_like(ids)
                for i, r in enumerate(rows):
                    ids[i, :r.numel()] = r
                    mask[i, :r.numel()] = 1
            labels = ids.masked_fill(mask == 0, -100)
            return {"input_ids": ids, "labels": labels, "attention_mask": mask}
        ids = torch.cat(rows).unsqueeze(0)
        total = ids.shape[1]
        bos = getattr(self.tokenizer, "bos_token_id", None)
        eos = getattr(self.tokenizer, "eos_token_id", None)
        if bos is not None:
            cuts = torch.nonzero(ids[0] == bos).flatten().tolist()
        elif eos is not None:
            cuts = (torch.nonzero(ids[0] == eos).flatten() + 1).tolist()
        else:
            raise ValueError("varlen batches need a tokenizer with a BOS or an EOS token to find document starts")
        bounds = sorted({0, total, *[c for c in cuts if 0 < c < total]})
        if self.context_len:
            split = set(bounds)
            for lo, hi in zip(bounds[:-1], bounds[1:]):
                split.update(range(lo, hi, int(self.context_len)))
            bounds = sorted(split)
        return {"input_ids": ids, "labels": ids.clone(), "cu_seqlens": torch.tensor(bounds, dtype=torch.int32)}


# ----------------------------------------------------------------------------- loader
def _identity(items):
    return items


class _WorkerDataset(torch.utils.data.IterableDataset):
    """The packer of one rank as an IterableDataset: every loader worker packs its own slice of the rank's samples."""

    def __init__(self, source, tokenizer, seq_len: int, rank: int, world: int, workers: int,
                 states: Optional[List[Dict[str, Any]]] = None):
        self.args = (source, tokenizer, seq_len, rank, world)
        self.workers, self.states = workers, states

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        wid = 0 if info is None else info.id
        packer = OnlineTokenizedPacker(*self.args, wid, self.workers)
        if self.states is not None and self.states[wid] is not None:
            packer.load_state_dict(self.states[wid])
        for item in packer:
            # the state AFTER this window travels with it, so the main process always knows where each worker is
            yield {"input_ids": item["input_ids"], "_worker": wid, "_state": packer.state_dict()}


class TextDataLoader:
    """Batches of packed windows for one data-parallel rank, optionally produced by worker processes.

    Resumable with any number of workers: every window carries its producer's state, ``state_dict()`` keeps the
    latest one per worker, and a restored loader restarts each worker from there (windows that a worker had
    prefetched beyond the last delivered batch are produced again, none is skipped or duplicated)."""

    def __init__(self, source, tokenizer, seq_len: int, batch_size: int, rank: int = 0, world: int = 1,
                 num_workers: int = 0, prefetch_factor: int = 2, pin_memory: bool = False,
                 persistent_workers: bool = False, varlen: bool = False, context_len: Optional[int] = None):
        self.source, self.tokenizer, self.seq_len, self.batch_size = source, tokenizer, seq_len, batch_size
        self.rank, self.world = rank, world
        self.num_workers = max(int(num_workers), 0)
        self.slots = max(self.num_workers, 1)
        self.prefetch_factor, self.persistent_workers = prefetch_factor, persistent_workers
        self.pin = bool(pin_memory) and torch.cuda.is_available()
        self.collate = LMCollator(tokenizer, context_len, varlen)
        if varlen and batch_size != 1:
            raise ValueError("training.varlen needs training.batch_size = 1 (rows are concatenated)")
        self.states: List[Optional[Dict[str, Any]]] = [None] * self.slots
        self._it = None

    def _start(self):
        ds = _WorkerDataset(self.source, self.tokenizer, self.seq_len, self.rank, self.world, self.slots,
                            copy.deepcopy(self.states))
        kwargs: Dict[str, Any] = {}
        if self.num_workers > 0:
            kwargs.update(prefetch_factor=self.prefetch_factor, persistent_workers=self.persistent_workers)
        loader = torch.utils.data.DataLoader(ds, batch_size=self.batch_size, num_workers=self.num_workers,
                                             collate_fn=_identity, **kwargs)
        self._it = iter(loader)

    def __iter__(self):
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        if self._it is None:
            self._start()
        items = next(self._it)
        for it in items:
            self.states[it["_worker"]] = it["_state"]
        batch = self.collate([{"input_ids": it["input_ids"]} for it in items])
        if self.pin:
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return batch

    def state_dict(self) -> Dict[str, Any]:
        return {"workers": copy.deepcopy(self.states), "num_workers": self.num_workers}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        if int(sd.get("num_workers", 0)) != self.num_workers:
            raise ValueError(f"the data position was saved with num_workers={sd.get('num_workers')} and cannot be "
                             f"restored with num_workers={self.num_workers} (each worker owns a slice of the samples)")
        self.states = copy.deepcopy(sd["workers"])
        self._it = None


def build_text_dataloader(dataset: str, *, tokenizer_path: Optional[str], seq_len: int, batch_size: int, rank: int,
                          world: int, seed: int = 0, dataset_name: Optional[str] = None, dataset_split: str = "train",
                          data_dir: Optional[str] = None, data_files: Optional[str] = None,
                          data_probs: Optional[str] = None, streaming: bool = False, num_workers: int = 0,
                          prefetch_factor: int = 2, pin_memory: bool = False, persistent_workers: bool = False,
                          varlen: bool = False, context_len: Optional[int] = None) -> TextDataLoader:
    """One dataset, or several comma-separated ones (names, splits, dirs and files then also comma-separated, with
    ``data_probs`` their mixing weights), as the reference's ``build_dataset`` takes them."""
    names = dataset.split(",")

    def nth(value: Optional[str], i: int) -> Optional[str]:
        if value is None:
            return None
        parts = value.split(",")
        return parts[i] if len(parts) == len(names) else value
    sources = [load_text_source(n, nth(dataset_name, i), nth(dataset_split, i) or "train", nth(data_dir, i),
                                nth(data_files, i), streaming, seed) for i, n in enumerate(names)]
    if len(sources) == 1:
        if data_probs:
            raise ValueError("training.data_probs needs more than one dataset")
        source = sources[0]
    else:
        if not data_probs:
            raise ValueError("several datasets need training.data_probs (their mixing weights)")
        probs = [float(p) for p in str(data_probs).split(",")]
        source = InterleavedSources(sources, probs, seed)
    return TextDataLoader(source, load_tokenizer(tokenizer_path), seq_len, batch_size, rank, world, num_workers,
                          prefetch_factor, pin_memory, persistent_workers, varlen, context_len)
