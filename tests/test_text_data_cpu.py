"""Text pipeline: online tokenisation + packing, rank / worker slicing, exact resume, interleave, collators."""
import json

import pytest
import torch

from uttt_b200.train.text_data import (ByteTokenizer, InterleavedSources, LMCollator, OnlineTokenizedPacker,
                                       TextDataLoader, _ListSource, build_text_dataloader)


def _docs(n, tag="doc"):
    return [{"text": f"{tag} {i}: " + "x" * (5 + (7 * i) % 23)} for i in range(n)]


def _take(it, n):
    return [next(it)["input_ids"].clone() for _ in range(n)]


def test_packer_concatenates_documents_and_resumes_exactly():
    tok = ByteTokenizer()
    src = _ListSource(_docs(40))
    full = _take(iter(OnlineTokenizedPacker(src, tok, 64)), 12)
    stream = torch.cat(full)
    want = torch.tensor(sum(tok([d["text"] for d in _docs(40)])["input_ids"], []))
    assert torch.equal(stream, want[:stream.numel()])                  # documents back to back, BOS ... EOS each
    p = OnlineTokenizedPacker(src, tok, 64)
    it = iter(p)
    first = _take(it, 5)
    state = p.state_dict()
    q = OnlineTokenizedPacker(src, tok, 64)
    q.load_state_dict(state)
    rest = _take(iter(q), 7)
    for a, b in zip(first + rest, full):
        assert torch.equal(a, b)


def test_pretokenized_rows_keep_their_length_and_epochs_wrap():
    tok = ByteTokenizer()
    src = _ListSource([{"input_ids": list(range(10))}, {"text": "ab"}, {"input_ids": [7] * 6}])
    p = OnlineTokenizedPacker(src, tok, 20)
    a, b = _take(iter(p), 2)
    assert a.tolist() == list(range(10)) + [256, 97, 98, 257] + [7] * 6
    assert b.tolist()[:10] == list(range(10)) and p.epoch >= 1           # the stream restarted


def test_ranks_and_workers_read_disjoint_slices():
    tok = ByteTokenizer()
    src = _ListSource([{"input_ids": [i] * 8} for i in range(24)])
    seen = {}
    for rank in range(2):
        for worker in range(2):
            p = OnlineTokenizedPacker(src, tok, 8, rank=rank, world=2, worker=worker, workers=2)
            seen[(rank, worker)] = {int(w[0]) for w in _take(iter(p), 6)}
    assert all(len(v) == 6 for v in seen.values())
    all_ids = set().union(*seen.values())
    assert all_ids == set(range(24)) and sum(len(v) for v in seen.values()) == 24


def test_interleave_follows_the_weights_and_is_seeded():
    a = _ListSource([{"input_ids": [0]}] * 50)
    b = _ListSource([{"input_ids": [1]}] * 50)
    mix = InterleavedSources([a, b], [3, 1], seed=4)
    it = iter(mix)
    first = [next(it)["input_ids"][0] for _ in range(2000)]
    assert 0.70 < first.count(0) / 2000 < 0.80
    it2 = iter(InterleavedSources([a, b], [3, 1], seed=4))
    assert first[:200] == [next(it2)["input_ids"][0] for _ in range(200)]
    with pytest.raises(ValueError):
        InterleavedSources([a, b], [1.0])


def test_collators():
    tok = ByteTokenizer()
    fixed = LMCollator(tok)([{"input_ids": torch.arange(6)}, {"input_ids": torch.arange(6) + 1}])
    assert fixed["input_ids"].shape == (2, 6) and torch.equal(fixed["labels"], fixed["input_ids"])
    padded = LMCollator(tok)([[1, 2, 3, 4], [5, 6]])
    assert padded["input_ids"][1].tolist() == [5, 6, 258, 258] and padded["labels"][1].tolist() == [5, 6, -100, -100]
    assert padded["attention_mask"][1].tolist() == [1, 1, 0, 0]
    row = [9, 9, 256, 1, 2, 3, 4, 5, 257, 256, 6, 257]
    var = LMCollator(tok, varlen=True)([row])
    assert var["input_ids"].shape == (1, 12) and var["cu_seqlens"].tolist() == [0, 2, 9, 12]
    var = LMCollator(tok, context_len=4, varlen=True)([row])
    assert var["cu_seqlens"].tolist() == [0, 2, 6, 9, 12]

    class EosOnly:
        bos_token_id, eos_token_id, pad_token_id = None, 257, None
    assert LMCollator(EosOnly(), varlen=True)([row])["cu_seqlens"].tolist() == [0, 9, 12]


@pytest.mark.parametrize("workers", [0, 2])
def test_json_files_through_datasets_with_workers_and_resume(tmp_path, workers):
    paths = []
    for f in range(4):
        path = tmp_path / f"part-{f}.jsonl"
        with open(path, "w") as fh:
            for d in _docs(30, tag=f"file{f}"):
                fh.write(json.dumps(d) + "\n")
        paths.append(str(path))
    kw = dict(tokenizer_path="byte", seq_len=48, batch_size=2, rank=1, world=2, seed=3,
              data_files=str(tmp_path / "part-*.jsonl"), num_workers=workers)
    loader = build_text_dataloader("json", **kw)
    assert isinstance(loader, TextDataLoader)
    batches = [next(loader) for _ in range(6)]
    assert batches[0]["input_ids"].shape == (2, 48) and torch.equal(batches[0]["labels"], batches[0]["input_ids"])
    state = loader.state_dict()
    after = [next(loader)["input_ids"] for _ in range(4)]
    resumed = build_text_dataloader("json", **kw)
    resumed.load_state_dict(json.loads(json.dumps(state)) if False else state)
    again = [next(resumed)["input_ids"] for _ in range(4)]
    # every window delivered after the resume point is delivered again, in the same per-worker order
    assert sorted(map(lambda t: t.flatten().tolist(), torch.cat(again))) == \
        sorted(map(lambda t: t.flatten().tolist(), torch.cat(after)))
    if workers == 0:
        for a, b in zip(again, after):
            assert torch.equal(a, b)
    with pytest.raises(ValueError):
        bad = build_text_dataloader("json", **{**kw, "num_workers": workers + 1})
        bad.load_state_dict(state)


def test_two_datasets_need_weights(tmp_path):
    for name in ("a", "b"):
        with open(tmp_path / f"{name}.jsonl", "w") as fh:
            for d in _docs(20, tag=name):
                fh.write(json.dumps(d) + "\n")
    files = f"{tmp_path}/a.jsonl,{tmp_path}/b.jsonl"
    with pytest.raises(ValueError):
        build_text_dataloader("json,json", tokenizer_path="byte", seq_len=32, batch_size=1, rank=0, world=1,
                              data_files=files)
    loader = build_text_dataloader("json,json", tokenizer_path="byte", seq_len=32, batch_size=1, rank=0, world=1,
                                   data_files=files, data_probs="0.5,0.5")
    assert next(loader)["input_ids"].shape == (1, 32)
