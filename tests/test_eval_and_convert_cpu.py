import math
import os

import pytest
import torch

from uttt_b200.config import named_config
from uttt_b200.eval.ptl import PerPositionLossTracker, evaluate, per_token_loss, summarize
from uttt_b200.eval.ruler import make_niah_sample, merge_shards, run_niah
from uttt_b200.models import build_model
from uttt_b200.train.checkpoint import CheckpointManager
from uttt_b200.train.data import PackedTokenDataset, SyntheticZipfTokens
from uttt_b200.utils.convert import dcp_to_hf, hf_to_dcp, preprocess
from uttt_b200.utils.flops import get_nparams_and_flops


def test_ptl_tracker_and_summary():
    t = PerPositionLossTracker(8)
    t.update(torch.ones(2, 8), torch.tensor([[1] * 6 + [0, 0]] * 2, dtype=torch.bool))
    m = t.mean()
    assert float(m[0]) == 1.0 and math.isnan(float(m[7]))
    s = summarize([1.0, 2.0, None, float("nan"), 4.0], start=1)
    assert s["ptl_tail_mean"] == 3.0 and s["tail_positions"] == 2


def test_ptl_matches_model_loss():
    torch.manual_seed(0)
    model = build_model(named_config("tiny-uttt-moe", memory_lb_loss_alpha=0.0)).eval()
    data = SyntheticZipfTokens(1024, 128, 2, seed=0)
    tracker = evaluate(model, data, 128, max_batches=1)
    data2 = SyntheticZipfTokens(1024, 128, 2, seed=0)
    ids = next(data2)["input_ids"]
    with torch.no_grad():
        want = model(input_ids=ids, labels=ids).ce_loss
    got = tracker.loss_sum.sum() / tracker.count.sum()
    assert abs(float(got) - float(want)) < 1e-4


def test_niah_sample_and_merge():
    s = make_niah_sample(1024, 256, 4, 3, seed=1)
    assert s["prompt"].shape == (256,) and int(s["prompt"][-3]) == 3
    key = int(s["prompt"][-2])
    pos = (s["prompt"][:-3] == key).nonzero()[0, 0]
    assert torch.equal(s["prompt"][pos + 2:pos + 5], s["answer"])
    model = build_model(named_config("tiny-uttt-moe")).eval()
    r0 = run_niah(model, 1024, 128, num_samples=2, num_needles=2, value_len=2, shard=0, num_shards=2)
    r1 = run_niah(model, 1024, 128, num_samples=2, num_needles=2, value_len=2, shard=1, num_shards=2)
    assert merge_shards([r0, r1])["total"] == 2


def test_convert_round_trip_and_preprocess(tmp_path):
    torch.manual_seed(0)
    cfg = named_config("tiny-uttt-moe")
    model = build_model(cfg)
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(cfg.to_json_string())
    mgr = CheckpointManager(str(tmp_path / "run"), interval=1)
    ck = mgr.save(5, model, force=True)
    hf = dcp_to_hf(ck, str(cfg_path), str(tmp_path / "hf"))
    assert os.path.exists(os.path.join(hf, "config.json"))
    back = hf_to_dcp(hf, str(tmp_path / "seed"))
    m2 = build_model(cfg)
    CheckpointManager(str(tmp_path / "seed")).load(m2)
    for (n, a), (_, b) in zip(model.state_dict().items(), m2.state_dict().items()):
        torch.testing.assert_close(a, b, msg=n)
    txt = tmp_path / "docs.txt"
    txt.write_text("\n".join(" ".join(str(i % 50) for i in range(j, j + 300)) for j in range(20)))
    shards = preprocess([str(txt)], str(tmp_path / "arrow"), lambda s: [int(x) for x in s.split()], shard_docs=8,
                        eos_token_id=2)
    assert len(shards) == 3
    ds = PackedTokenDataset(shards, seq_len=64, batch_size=2, pin=False)
    b = next(ds)
    assert b["input_ids"].shape == (2, 64)
    st = ds.state_dict()
    nxt = next(ds)["input_ids"]
    ds.load_state_dict(st)
    torch.testing.assert_close(next(ds)["input_ids"], nxt)


def test_flop_model_subtracts_embeddings():
    cfg = named_config("tiny-uttt-moe")
    model = build_model(cfg)
    n, flops = get_nparams_and_flops(model, cfg, 256)
    assert n == sum(p.numel() for p in model.parameters())
    assert flops < 6 * n + 12 * 2 * 4 * 16 * 256 + 1e9 and flops > 6 * (n - 1024 * 64 * 2)


def test_validation_loss_and_offload_context_cpu():
    import torch
    from uttt_b200.config import named_config
    from uttt_b200.eval.validate import validation_loss
    from uttt_b200.models import build_model
    from uttt_b200.train.data import SyntheticZipfTokens
    from uttt_b200.utils.activation_offload import offload_activations
    cfg = named_config("tiny-uttt-moe")
    model = build_model(cfg)
    out = validation_loss(model, SyntheticZipfTokens(cfg.vocab_size, 128, 2, seed=3), max_batches=2)
    assert out["tokens"] == 2 * 2 * 127 and 0 < out["loss"] < 20 and out["perplexity"] > 1
    # on CPU tensors the offloading context changes nothing
    lin = torch.nn.Linear(8, 8)
    x = torch.randn(4, 8, requires_grad=True)
    with offload_activations(min_bytes=0) as off:
        y = lin(x).relu().sum()
    y.backward()
    assert off.tensors_offloaded == 0 and x.grad is not None


def test_ptl_job_file_interface_and_summary_tool(tmp_path, capsys):
    """The job-file interface writes the flat per-position list under the reference's file name; the summary tool
    reduces it with the published rule (NaN-aware mean from a 0-based first position) and the reference's keys."""
    import json
    import math
    from uttt_b200.config import named_config
    from uttt_b200.eval import ptl
    from uttt_b200.models import build_model
    from uttt_b200.train.checkpoint import export_hf
    cfg = named_config("tiny-uttt-moe")
    torch.manual_seed(0)
    model = build_model(cfg)
    export_hf(model, cfg, str(tmp_path / "hf"))
    job = tmp_path / "eval.toml"
    job.write_text('[job]\ndump_folder = "%s"\n[training]\nbatch_size = 1\nseq_len = 256\nsteps = 2\n'
                   'dataset = "synthetic"\n[eval]\nper_token_loss_from_hidden = true\nlm_head_chunk_size = 64\n'
                   % (tmp_path / "out"))
    assert ptl.main(["--job.config_file", str(job), "--checkpoint.load_path", str(tmp_path / "hf"),
                     "--training.save_prefix", "tiny"]) == 0
    path = tmp_path / "out" / "tiny_loss_per_token_position.json"
    data = json.loads(path.read_text())
    assert isinstance(data, list) and len(data) == 256 and data[-1] is None and all(v > 0 for v in data[:-1])
    capsys.readouterr()
    assert ptl.main(["summarize", str(path), "--min-position", "200", "--expect-positions", "256", "--chunks", "4",
                     "--output", str(tmp_path / "s.json")]) == 0
    out = capsys.readouterr().out
    assert "PTL(>= 200)" in out and "1 NaN position(s) skipped" in out and "blocks:" in out
    s = json.loads((tmp_path / "s.json").read_text())[str(path)]
    assert set(s) == {"positions", "min_position", "tail_positions", "tail_nan", "ptl", "mean_all", "chunk_means"}
    assert s["positions"] == 256 and s["tail_positions"] == 56 and s["tail_nan"] == 1 and len(s["chunk_means"]) == 4
    assert s["ptl"] == pytest.approx(sum(data[200:-1]) / 55)
    assert s["chunk_means"][3] == pytest.approx(sum(data[192:-1]) / 63)
    both = ptl.summarize_positions([1.0, math.nan, 3.0, 5.0], 1)
    assert both["ptl"] == 4.0 and both["mean_all"] == 3.0 and both["tail_nan"] == 1
    with pytest.raises(ValueError):
        ptl.summarize_positions([1.0], 1)
    (tmp_path / "bad.json").write_text('["a"]')
    with pytest.raises(ValueError):
        ptl.load_positions(tmp_path / "bad.json")
    (tmp_path / "obj.json").write_text(json.dumps({"per_position_loss": [1.0, None], "count": [2, 0]}))
    assert ptl.load_positions(tmp_path / "obj.json")[0] == 1.0


class _ByteTokenizer:
    eos_token_id = 0

    def encode(self, text):
        return [b + 1 for b in text.encode("utf-8")]

    def decode(self, ids):
        return bytes(max(i - 1, 0) % 256 for i in ids).decode("latin-1")


def test_harness_adapter_requests_and_shard_bookkeeping(tmp_path):
    """The three request kinds of the evaluation harness on a tiny model, without the harness package."""
    import json
    from types import SimpleNamespace
    from uttt_b200.eval import harness
    from uttt_b200.models.generation import generate
    torch.manual_seed(0)
    model = build_model(named_config("tiny-uttt-moe", memory_lb_loss_alpha=0.0)).eval()
    tok = _ByteTokenizer()
    adapter = harness.TextAdapter(model, tok, max_length=96, device="cpu")
    prompt = "needle 42 is hidden here. " * 3
    # greedy continuation equals the package's own generate()
    ids = torch.tensor([tok.encode(prompt)])
    want = generate(model, ids, max_new_tokens=6)[0, ids.shape[1]:].tolist()
    if 0 in want:
        want = want[:want.index(0)]
    got = adapter.generate_until([SimpleNamespace(args=(prompt, {"until": [], "max_gen_toks": 6}))])
    assert got == [tok.decode(want)]
    # a stop string ends the text before it
    full = tok.decode(want)
    if len(full) >= 3:
        stop = full[2]
        cut = adapter.generate_until([(prompt, {"until": [stop], "max_gen_toks": 6})])[0]
        assert cut == full[:full.find(stop)]
    assert harness.first_stop("abc\n\ndef", ["\n\n", "f"]) == "abc" and harness.first_stop("abc", []) == "abc"
    # log-likelihood equals the sum of next-token log-probabilities of a plain forward
    cont = " 42"
    (ll, greedy), = adapter.loglikelihood([(prompt, cont)])
    seq = tok.encode(prompt) + tok.encode(cont)
    with torch.no_grad():
        logits = model(input_ids=torch.tensor([seq[:-1]])).logits[0].float()
    logp = torch.log_softmax(logits, -1)
    n = len(tok.encode(cont))
    ref = sum(float(logp[len(seq) - 1 - n + j, seq[len(seq) - n + j]]) for j in range(n))
    assert ll == pytest.approx(ref, abs=1e-3) and isinstance(greedy, bool)
    rolling = adapter.loglikelihood_rolling([(prompt,)])[0]
    assert math.isfinite(rolling) and rolling < 0
    # strided shards and their manifest
    none, off = harness.strided_samples({"niah": 10}, 0, 1)
    assert none is None and off["enabled"] is False
    picks, manifest = harness.strided_samples({"niah": 10, "vt": 3}, 1, 4)
    assert picks == {"niah": [1, 5, 9], "vt": [1]}
    assert manifest["tasks"]["niah"] == {"total_samples": 10, "shard_samples": 3, "first_index": 1, "last_index": 9}
    with pytest.raises(ValueError):
        harness.strided_samples({"niah": 10}, 4, 4)
    with pytest.raises(ValueError):
        harness.strided_samples({"niah": 2}, 3, 4)
    # shard results pooled by sample count
    for r, (score, count) in enumerate(((1.0, 3), (0.0, 1))):
        folder = tmp_path / "shards" / f"shard_{r}"
        folder.mkdir(parents=True)
        (folder / "results.json").write_text(json.dumps({
            "results": {"niah": {"4096,none": score, "4096_stderr,none": 0.1, "alias": "niah"}},
            "sample_shard": {"enabled": True, "rank": r, "world_size": 2,
                             "tasks": {"niah": {"shard_samples": count}}}}))
    assert harness.main(["merge", "--shards-dir", str(tmp_path / "shards"), "--output-dir", str(tmp_path / "merged"),
                         "--expected-shards", "2"]) == 0
    merged = json.loads((tmp_path / "merged" / "results.json").read_text())
    assert merged["results"]["niah"] == {"4096,none": 0.75} and merged["samples_per_task"] == {"niah": 4.0}
    assert harness.main(["merge", "--shards-dir", str(tmp_path / "shards"), "--output-dir", str(tmp_path / "m2"),
                         "--expected-shards", "3"]) == 1
    assert harness.write_samples({"a/b": [{"x": 1}]}, tmp_path) == ["samples/a_b.jsonl"]
    try:
        import lm_eval  # noqa: F401
    except ImportError:                                   # the command says what to run instead
        assert harness.main(["--model-dir", str(tmp_path), "--output", str(tmp_path / "r.json")]) == 2
