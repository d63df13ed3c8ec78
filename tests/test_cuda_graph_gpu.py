"""Forward + backward replayed from a CUDA graph must give the gradients of the eager step.

The engine captures the first step after its warm-up and replays it afterwards; the optimizer stays eager.  The
kernels and their order are identical, only the launch mechanism differs.  A routed model at random initialisation
is not bit-reproducible from run to run (fp32 atomics move a few bf16 roundings, near-tied router logits then pick
other experts), so the comparison is calibrated: the graph's gradients must be as close to an eager run's as a second
eager run is."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TINY = dict(hidden_size=256, num_heads=4, fw_num_heads=2, memory_num_experts=4, memory_num_active_experts=2,
            chunk_size=128, window_size=128)


def _engine(graph, **over):
    from uttt_b200.config import named_config
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    cfg = named_config("tiny-uttt-moe", **{**TINY, **over})
    return cfg, TrainEngine(cfg, EngineConfig(micro_batch_size=2, lr=1e-3, eps=1e-6, warmup_steps=0, total_steps=100,
                                              seed=0, cuda_graph=graph, cuda_graph_warmup=2), torch.device("cuda", 0))


def _take_grads(eng):
    out = {}
    for u in eng.trainer.units:
        for s in u.slots:
            out[s.name] = u.grad[s.offset:s.offset + s.numel].float().clone()
        u.grad.zero_()
    return out


def _rel(a, b):
    return float((a - b).norm() / b.norm().clamp_min(1e-20))


@pytest.mark.parametrize("over", [dict(), dict(memory_lb_mode="loss_free", memory_loss_free_update_rate=1e-2),
                                  dict(memory_num_experts=1, memory_num_active_experts=1)])
def test_graph_replay_gives_the_eager_gradients(over):
    cfg, eng = _engine(True, **over)
    dev = eng.device
    ids = torch.randint(0, cfg.vocab_size, (2, 4 * cfg.chunk_size), generator=torch.Generator().manual_seed(3)).to(dev)
    eng.model.train()

    def eager():
        out = eng.model(input_ids=ids, labels=ids)
        out.loss.backward()
        return float(out.loss.detach()), _take_grads(eng)

    loss_a, grads_a = eager()
    loss_b, grads_b = eager()
    eng.step = eng.cfg.cuda_graph_warmup
    out = eng._replay_forward_backward(ids, ids, 1)
    assert out is not None and eng.graph_error is None, eng.graph_error
    loss_g, grads_g = float(out.loss), _take_grads(eng)
    out = eng._replay_forward_backward(ids, ids, 1)           # a second replay of the same graph
    loss_h, grads_h = float(out.loss), _take_grads(eng)
    assert len(eng._graphs) == 1
    noise_loss = abs(loss_a - loss_b)
    assert abs(loss_g - loss_a) <= 3 * noise_loss + 1e-4 * abs(loss_a), (loss_a, loss_b, loss_g)
    assert abs(loss_h - loss_a) <= 3 * noise_loss + 1e-4 * abs(loss_a), (loss_a, loss_b, loss_h)
    for name, g in grads_a.items():
        if g.numel() < 64:                       # one-element biases: sums that cancel, all rounding
            continue
        if float(g.norm()) == 0.0:
            assert float(grads_g[name].norm()) == 0.0, name
            continue
        noise = _rel(grads_b[name], g)
        for got in (grads_g[name], grads_h[name]):
            assert _rel(got, g) <= 3.0 * noise + 5e-2, (name, _rel(got, g), noise)


def test_graph_replay_trains_and_keeps_the_host_side_bookkeeping():
    from uttt_b200 import ops
    cfg, eng = _engine(True, memory_lb_mode="loss_free", memory_loss_free_update_rate=1e-2)
    _, ref = _engine(False, memory_lb_mode="loss_free", memory_loss_free_update_rate=1e-2)
    g = torch.Generator().manual_seed(7)
    inner = eng.model.model
    bias_before = inner.memory_loss_free_bias.clone()
    for step in range(5):
        ids = torch.randint(0, cfg.vocab_size, (2, 4 * cfg.chunk_size), generator=g)
        before = ops.launch_count()
        loss = float(eng.train_step({"input_ids": ids, "labels": ids}))
        launched = ops.launch_count() - before
        want = float(ref.train_step({"input_ids": ids, "labels": ids}))
        assert abs(loss - want) <= 5e-3 * abs(want), (step, loss, want)
        if step >= 2:
            sg = next(iter(eng._graphs.values()))
            assert sg.launches > 0 and launched >= sg.launches       # replayed launches are counted
            # the replayed forward moved the balancing bias (+-rate per expert, re-centred) like an eager one
            assert not torch.equal(inner.memory_loss_free_bias, bias_before), step
        bias_before = inner.memory_loss_free_bias.clone()
    assert eng.graph_error is None, eng.graph_error
    assert len(eng._graphs) == 1                                     # one capture, replayed by every later step
    assert int(inner.memory_loss_free_steps) == 5 and inner._host_steps == 5
    assert int(inner.memory_loss_free_num_updates) == int(ref.model.model.memory_loss_free_num_updates) == 4


def test_recomputation_reuses_the_attention_output(monkeypatch):
    """A checkpointed region keeps its attention output (and its routing and group layout) from the first pass and
    its recomputation takes them back: at least one launch fewer per (chunk, layer) and step, same loss."""
    from uttt_b200 import ops
    results = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("UTTT_B200_REUSE_ATTENTION", flag)
        cfg, eng = _engine(False, memory_num_experts=1, memory_num_active_experts=1)
        ids = torch.randint(0, cfg.vocab_size, (2, 4 * cfg.chunk_size), generator=torch.Generator().manual_seed(5))
        before = ops.launch_count()
        loss = float(eng.train_step({"input_ids": ids, "labels": ids}))
        results[flag] = (loss, ops.launch_count() - before)
        for layer in eng.model.model.layers:
            assert not layer.attn.reuse_store                      # every kept output was taken back
    regions = 4 * cfg.num_hidden_layers                            # chunks x layers
    assert results["0"][1] - results["1"][1] >= regions, results
    assert abs(results["0"][0] - results["1"][0]) <= 1e-4 * abs(results["0"][0]), results


def test_recomputation_takes_the_write_aggregate_back(monkeypatch):
    """The aggregate of a chunk write is kept from the first pass; the recomputation records the writers' nodes
    without their GEMMs and reductions.  Gradients must be those of the full recomputation (up to the run-to-run
    noise of a routed model, measured by repeating the reference run)."""
    grads = {}
    for name, flag in (("full_a", "0"), ("full_b", "0"), ("kept", "1")):
        monkeypatch.setenv("UTTT_B200_REUSE_AGGREGATE", flag)
        cfg, eng = _engine(False)
        ids = torch.randint(0, cfg.vocab_size, (2, 4 * cfg.chunk_size),
                            generator=torch.Generator().manual_seed(11)).to(eng.device)
        eng.model.train()
        out = eng.model(input_ids=ids, labels=ids)
        out.loss.backward()
        assert not eng.model.model._aggregate_store            # every kept aggregate was taken back (or none kept)
        grads[name] = (float(out.loss.detach()), _take_grads(eng))
    assert abs(grads["kept"][0] - grads["full_a"][0]) <= 1e-4 * abs(grads["full_a"][0])
    for k, g in grads["full_a"][1].items():
        if g.numel() < 64 or float(g.norm()) == 0.0:
            continue
        noise = _rel(grads["full_b"][1][k], g)
        assert _rel(grads["kept"][1][k], g) <= 3.0 * noise + 5e-2, (k, _rel(grads["kept"][1][k], g), noise)


def test_dense_family_keeps_its_write_aggregate_too(monkeypatch):
    """uTTT-Dense: stashed token reductions and the kept aggregate give the gradients of the plain recomputation, as
    closely as a second plain run does (Newton-Schulz on bf16 copies amplifies the last-bit differences of two
    summation orders, so even the dense family is not bit-reproducible)."""
    from uttt_b200.config import named_config
    from uttt_b200.train.engine import EngineConfig, TrainEngine
    out = {}
    for name, reuse, stash in (("plain_a", "0", "1"), ("plain_b", "0", "1"), ("kept", "1", "4")):
        monkeypatch.setenv("UTTT_B200_REUSE_AGGREGATE", reuse)
        monkeypatch.setenv("UTTT_B200_WRITE_STASH", stash)
        cfg = named_config("124M-uttt-dense", num_hidden_layers=3, vocab_size=2048, chunk_size=256, window_size=256)
        eng = TrainEngine(cfg, EngineConfig(micro_batch_size=2, warmup_steps=0, total_steps=10, seed=0),
                          torch.device("cuda", 0))
        ids = torch.randint(0, cfg.vocab_size, (2, 4 * cfg.chunk_size),
                            generator=torch.Generator().manual_seed(2)).to(eng.device)
        eng.model.train()
        res = eng.model(input_ids=ids, labels=ids)
        res.loss.backward()
        assert not eng.model.model._aggregate_store
        grads = _take_grads(eng)
        out[name] = (float(res.loss.detach()), torch.cat([g.reshape(-1) for g in grads.values()]))
    assert abs(out["plain_a"][0] - out["kept"][0]) <= 1e-4 * abs(out["plain_a"][0]), (out["plain_a"][0], out["kept"][0])
    noise = _rel(out["plain_b"][1], out["plain_a"][1])
    got = _rel(out["kept"][1], out["plain_a"][1])
    assert got <= 3.0 * noise + 1e-2, (got, noise)
