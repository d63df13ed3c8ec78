"""CPU plumbing run of the tiny uTTT-MoE LM: forward/backward, one AdamW step through the
sharded engine, checkpoint save/load round trip (fp32, seed 0)."""
import copy

import torch

from uttt_b200.config import named_config
from uttt_b200.models import build_model
from uttt_b200.train.checkpoint import CheckpointManager, TrainState
from uttt_b200.train.engine import EngineConfig, TrainEngine


def _batch(seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 1024, (2, 256), generator=g)
    return {"input_ids": ids, "labels": ids}


def test_forward_backward_all_params_get_grads():
    torch.manual_seed(0)
    model = build_model(named_config("tiny-uttt-moe"))
    out = model(**_batch())
    assert abs(out.ce_loss.item() - 6.93) < 0.3
    out.loss.backward()
    for name, p in model.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        assert p.grad.abs().sum() > 0, name


def test_chunking_is_causal():
    """Changing a late token must not change the hidden state of earlier positions."""
    torch.manual_seed(0)
    model = build_model(named_config("tiny-uttt-moe")).eval()
    b = _batch()
    with torch.no_grad():
        h1 = model(input_ids=b["input_ids"]).hidden_states
        ids2 = b["input_ids"].clone()
        ids2[:, 200] = (ids2[:, 200] + 1) % 1024
        h2 = model(input_ids=ids2).hidden_states
    torch.testing.assert_close(h1[:, :200], h2[:, :200], atol=1e-5, rtol=1e-5)
    assert (h1[:, 200:] - h2[:, 200:]).abs().max() > 1e-4


def test_memory_write_changes_later_chunks():
    """With the write disabled (lr -> 0) later chunks differ: the bank carries information."""
    torch.manual_seed(0)
    cfg = named_config("tiny-uttt-moe")
    model = build_model(cfg).eval()
    b = _batch()
    with torch.no_grad():
        h1 = model(input_ids=b["input_ids"]).hidden_states
        for layer in model.model.layers:
            layer.base_lr_inv = -50.0
        h2 = model(input_ids=b["input_ids"]).hidden_states
    torch.testing.assert_close(h1[:, :64], h2[:, :64])        # first chunk reads the initial bank
    assert (h1[:, 64:] - h2[:, 64:]).abs().max() > 1e-5


def test_train_step_and_checkpoint_roundtrip(tmp_path):
    cfg = named_config("tiny-uttt-moe")
    eng = TrainEngine(cfg, EngineConfig(micro_batch_size=2, lr=1e-3, warmup_steps=0, total_steps=10, seed=0))
    loss0 = float(eng.train_step(_batch(0)))
    loss1 = float(eng.train_step(_batch(0)))
    assert loss1 < loss0
    mgr = CheckpointManager(str(tmp_path), interval=1, keep_latest_k=2)
    ts = TrainState(step=2, token=1024)
    path = mgr.save(2, eng.model, eng.trainer, eng.lr_sched, train_state=ts)
    assert path is not None and mgr.steps() == [2]
    want = float(eng.train_step(_batch(1)))

    eng2 = TrainEngine(cfg, EngineConfig(micro_batch_size=2, lr=1e-3, warmup_steps=0, total_steps=10, seed=123))
    ts2 = TrainState()
    step = mgr.load(eng2.model, eng2.trainer, eng2.lr_sched, train_state=ts2)
    assert step == 2 and ts2.token == 1024
    got = float(eng2.train_step(_batch(1)))
    assert abs(got - want) < 1e-5
    for (n1, p1), (n2, p2) in zip(eng.model.named_parameters(), eng2.model.named_parameters()):
        torch.testing.assert_close(p1, p2, atol=1e-6, rtol=1e-5, msg=n1)


def test_state_dict_keys_follow_reference_layout():
    model = build_model(named_config("tiny-uttt-moe"))
    keys = set(model.state_dict().keys())
    for k in ("model.embeddings.weight", "model.layers.0.attn_norm.weight", "model.layers.0.attn.q_proj.weight",
              "model.layers.0.memory.qk_scale", "model.layers.0.memory.momentum_proj.0.weight",
              "model.layers.0.memory.ttt_norm.weight", "model.layers.0.memory.ttt_scale_proj.bias",
              "model.layers.0.to_lr.weight", "model.layers.0.memory_output_proj.weight",
              "model.layers.0.mlp.gate_proj.weight", "model.norm.weight", "model.pool_w0", "model.pool_w1",
              "model.per_layer_router_proj_weights", "model.memory_loss_free_bias", "lm_head.weight"):
        assert k in keys, k
    lowrank = build_model(named_config("tiny-uttt-moe", w0_w2_low_rank=8))
    assert "model.pool_w0.w_left" in lowrank.state_dict() and "model.pool_w2.w_right" in lowrank.state_dict()
