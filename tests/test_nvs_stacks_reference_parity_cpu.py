"""The dense fast-weight stacks, the delta-rule baselines and the key/value-cache transformer of the view-synthesis
model against the reference's own modules, on the CPU.

These reference stacks are plain PyTorch (no Triton), so they run here: ``uttt_nvs.models.{ttt_dense_block,
uttt_dense_block, uttt_dense_partitioned, deltanet_block, gated_deltanet_block, transformer_block}.MemoryModel`` from
the verbatim copy under ``baseline/_ref/uttt_nvs`` (not part of this repository's history).  Around them only:
``torch.compile`` is switched off (``TORCH_COMPILE_DISABLE``), matplotlib gets the stand-in of the reference arm, and
``flash_attn_func`` (CUDA only) is replaced by softmax attention.  Both sides get the same state dict (strict load: the
layouts are identical), the same tokens and schedule, and run under bf16 autocast as the trainers run them.
Compared: the output tokens and the gradients of every parameter.  Skipped when the reference tree is absent.
"""
import importlib
import os
import sys

import pytest
import torch

from uttt_b200.nvs import stacks
from uttt_b200.nvs.schedule import TTTConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "uttt_nvs", "models")),
                                reason="reference tree (baseline/_ref/uttt_nvs) not present")

DIM, TOK = 64, 16


def _attention_stand_in(q, k, v, *args, **kwargs):
    """q [b, lq, h, d], k / v [b, lk, h, d], no mask."""
    o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2)


def _reference(module: str):
    os.environ["TORCH_COMPILE_DISABLE"] = "1"
    import torch._dynamo
    torch._dynamo.config.disable = True
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import run_reference as rr
    rr._nvs_stand_ins()
    if REF not in sys.path:
        sys.path.insert(0, REF)
    if module == "transformer_block":
        import flash_attn
        flash_attn.flash_attn_func = _attention_stand_in
    mod = importlib.import_module(f"uttt_nvs.models.{module}")
    if module == "transformer_block":
        mod.flash_attn_func = _attention_stand_in
    return mod.MemoryModel


def _schedule(views: int = 3):
    """input view (read + write), target view (read), ..., as the decoder's schedule alternates them."""
    cfg, pos = [], 0
    for _ in range(views):
        cfg.append(TTTConfig(pos, pos + TOK, True, True, True))
        cfg.append(TTTConfig(pos + TOK, pos + 2 * TOK, False, False, True))
        pos += 2 * TOK
    return cfg, pos


CASES = [
    ("ttt_dense_block", stacks.TTTDenseModel,
     dict(attn_head_dim=16, fw_head_dim=16, inter_multi=2, fw_inter_multi=2, l2_norm=True, use_muon=False)),
    ("ttt_dense_block", stacks.TTTDenseModel,
     # Newton-Schulz lifts every singular value towards one, rounding noise in a null space included: the heads are
     # kept smaller (8 x 8) than the number of tokens of a view so that the steps have full rank.  Even so, two bf16
     # evaluations of the five iterations that differ only in the order of their roundings are 3 % apart
     # (`test_newton_schulz_spread`), and the stack chains twelve of them: this case gets the wide bounds.
     dict(attn_head_dim=16, fw_head_dim=8, inter_multi=2, fw_inter_multi=1, l2_norm=False, use_muon=True, v_gap=1)),
    ("uttt_dense_block", stacks.UTTTDenseModel,
     dict(attn_head_dim=16, fw_head_dim=16, inter_multi=3, fw_inter_multi=4, l2_norm=True, use_muon=False,
          aggregate_write=True)),
    ("uttt_dense_block", stacks.UTTTDenseModel,
     dict(attn_head_dim=16, fw_head_dim=16, inter_multi=2, fw_inter_multi=2, l2_norm=True, use_muon=False,
          aggregate_write=False, v_gap=-1)),
    ("uttt_dense_partitioned", stacks.UTTTDensePartitionedModel,
     dict(attn_head_dim=16, fw_head_dim=16, inter_multi=2, fw_inter_multi=2, l2_norm=True, use_muon=False,
          aggregate_write=True, num_shared_pools=2)),
    ("uttt_dense_partitioned", stacks.UTTTDensePartitionedModel,
     dict(attn_head_dim=16, fw_head_dim=16, inter_multi=2, fw_inter_multi=1, l2_norm=True, use_muon=False,
          aggregate_write=False, num_shared_pools=4)),
    ("deltanet_block", stacks.DeltaNetModel,
     dict(attn_head_dim=16, fw_num_heads=4, inter_multi=3.09375, expand_k=1.0, expand_v=1.0, use_beta=True,
          noise_repeat=1, repeat_function="repeat", use_muon=False, conv_size=4, conv_bias=False, qk_activation="silu",
          qk_norm="l2", use_output_gate=False, allow_neg_eigval=False, use_short_conv=False)),
    ("deltanet_block", stacks.DeltaNetModel,
     dict(attn_head_dim=16, fw_num_heads=2, inter_multi=2, expand_v=2.0, use_beta=True, noise_repeat=2,
          repeat_function="repeat", qk_activation="elu", qk_norm="sum", use_output_gate=True, allow_neg_eigval=True,
          use_short_conv=True, bias=True, v_gap=1)),
    ("gated_deltanet_block", stacks.GatedDeltaNetModel,
     dict(attn_head_dim=16, fw_num_heads=4, inter_multi=2.75, expand_v=1.0, noise_repeat=1, repeat_function="repeat",
          use_muon=False, conv_size=4, conv_bias=False, use_output_gate=True, use_short_conv=False)),
    ("gated_deltanet_block", stacks.GatedDeltaNetModel,
     dict(attn_head_dim=16, fw_num_heads=2, inter_multi=2, expand_v=2.0, repeat_function="linear", use_short_conv=True,
          conv_bias=True, use_output_gate=False)),
    ("transformer_block", stacks.TransformerModel,
     dict(attn_head_dim=16, inter_multi=3, transformer_version="v0", vi_rms_norm=True, pre_vi_source="xi_memory_in",
          use_separate_last_to_kv=False)),
    ("transformer_block", stacks.TransformerModel,
     dict(attn_head_dim=16, inter_multi=2, transformer_version="v1", to_kv_mode="per_layer", bias=True)),
    ("transformer_block", stacks.TransformerModel,
     dict(attn_head_dim=16, inter_multi=2, transformer_version="v3", use_separate_last_to_kv=True, v_gap=1,
          pre_vi_source="xi_out")),
    ("transformer_block", stacks.TransformerModel,
     dict(attn_head_dim=16, inter_multi=2, transformer_version="v4", to_kv_mode="shared_last")),
]


@pytest.mark.parametrize("module,ours_cls,params", CASES,
                         ids=[f"{m}-{i}" for i, (m, _, _) in enumerate(CASES)])
def test_stack_matches_the_reference(module, ours_cls, params):
    ref_cls = _reference(module)
    layers = 4
    torch.manual_seed(0)
    ref = ref_cls(layers=layers, dim=DIM, **params)
    ours = ours_cls(layers=layers, dim=DIM, **params)
    res = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    assert {k: tuple(v.shape) for k, v in ours.state_dict().items()} == \
           {k: tuple(v.shape) for k, v in ref.state_dict().items()}
    sched, length = _schedule()
    x = torch.randn(2, length, DIM)
    xr, xo = x.clone().requires_grad_(), x.clone().requires_grad_()
    probe = torch.randn(2, length, DIM)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        out_r = ref(xr, {"ttt_config": [tuple(c) for c in sched], "num_img_tokens": TOK})[0]
        out_o = ours(xo, {"ttt_config": sched, "num_img_tokens": TOK})[0]
    assert out_o.shape == out_r.shape
    scale = out_r.float().abs().mean()
    err = (out_o.float() - out_r.float()).abs().mean() / scale
    if params.get("use_muon"):
        # calibrated against the reference's own sensitivity: its output under a 0.1 % perturbation of the tokens.
        # The gradients through twelve chained orthogonalisations decorrelate under that perturbation (cosine 0.3 on
        # this case), so they are compared on the cases without Newton-Schulz only.
        with torch.no_grad(), torch.autocast("cpu", dtype=torch.bfloat16):
            moved = ref(x * (1 + 1e-3 * torch.randn_like(x)), {"ttt_config": [tuple(c) for c in sched]})[0]
        spread = (moved.float() - out_r.float()).abs().mean() / scale
        assert err < 2 * spread, f"outputs differ by {err:.3f}; the reference moves by {spread:.3f} on its own"
        return
    assert err < 0.02, f"outputs differ: mean |d| / mean |ref| = {err:.4f}"
    (out_r.float() * probe).sum().backward()
    (out_o.float() * probe).sum().backward()
    cos = torch.nn.functional.cosine_similarity(xo.grad.flatten(), xr.grad.flatten(), dim=0)
    assert cos > 0.995, f"input gradient: cosine {cos:.4f}"
    ref_grads = dict(ref.named_parameters())
    worst = 1.0
    for name, p in ours.named_parameters():
        g_r = ref_grads[name].grad
        if g_r is None:                                     # a parameter that nothing read in the reference either
            assert p.grad is None or p.grad.abs().max() == 0, name
            continue
        assert p.grad is not None, name
        if g_r.abs().max() == 0:
            continue
        c = torch.nn.functional.cosine_similarity(p.grad.flatten().float(), g_r.flatten().float(), dim=0)
        worst = min(worst, float(c))
        assert c > 0.97, f"{name}: gradient cosine {c:.4f}"


def test_newton_schulz_spread():
    """The reference's Newton-Schulz routine against this package's on the same bf16 inputs: the same five iterations,
    a different order of roundings.  The gap is a few per cent; fp32 iterations are as far from either."""
    _reference("ttt_dense_block")
    from uttt_nvs.models.ttt_dense_block import zeropower_via_newtonschulz5
    from uttt_b200.ops import reference as plain
    torch.manual_seed(0)
    for shape in ((6, 8, 8), (6, 8, 16), (6, 16, 8)):
        g = (torch.randn(*shape) * 1e-3).bfloat16()
        theirs = zeropower_via_newtonschulz5(g, 5).float()
        ours = plain.newton_schulz(g.float(), plain.NS_FIXED_COEFFS, compute_dtype=torch.bfloat16).float()
        exact = plain.newton_schulz(g.double(), plain.NS_FIXED_COEFFS, compute_dtype=torch.float64).float()
        assert theirs.shape == ours.shape == g.shape
        gap = (theirs - ours).abs().mean() / theirs.abs().mean()
        assert gap < 0.08
        assert (ours - exact).abs().mean() / exact.abs().mean() < 0.08
        assert (theirs - exact).abs().mean() / exact.abs().mean() < 0.08


def test_fp32_run_is_close_to_the_autocast_run():
    """Without autocast the stacks compute in the activations' precision; the bf16 run stays near it."""
    torch.manual_seed(1)
    model = stacks.UTTTDenseModel(layers=2, dim=DIM, attn_head_dim=16, fw_head_dim=16, fw_inter_multi=2, l2_norm=True,
                                  use_muon=False, aggregate_write=True)
    sched, length = _schedule(2)
    x = torch.randn(1, length, DIM)
    with torch.no_grad():
        full = model(x, {"ttt_config": sched})[0]
        with torch.autocast("cpu", dtype=torch.bfloat16):
            low = model(x, {"ttt_config": sched})[0]
    assert full.dtype == torch.float32
    assert (full - low.float()).abs().mean() / full.abs().mean() < 0.02


def test_every_reference_configuration_builds_with_the_reference_state_dict_layout():
    """Each YAML file the reference ships, read unchanged: this package's model and the reference's own, built on the
    meta device, must have the same state-dict keys with the same shapes (so its checkpoints load strictly)."""
    import glob
    import yaml
    _reference("transformer_block")                       # stand-ins in place, every family importable
    from easydict import EasyDict
    from uttt_b200.nvs.model import LVSMModel
    files = sorted(glob.glob(os.path.join(REF, "uttt_nvs", "configs", "**", "*.yaml"), recursive=True))
    assert len(files) >= 70
    for path in files:
        with open(path) as fh:
            cfg = yaml.safe_load(fh)
        cfg["training"].update(perceptual_loss_weight=0.0, lpips_loss_weight=0.0)    # their networks need downloads
        module, name = cfg["model"]["class_name"].rsplit(".", 1)
        with torch.device("meta"):
            theirs = getattr(importlib.import_module(module), name)(EasyDict(cfg))
            ours = LVSMModel(cfg)
        a = {k: tuple(v.shape) for k, v in theirs.state_dict().items()}
        b = {k: tuple(v.shape) for k, v in ours.state_dict().items()}
        rel = os.path.relpath(path, REF)
        assert sorted(set(a) - set(b)) == [] and sorted(set(b) - set(a)) == [], rel
        assert a == b, rel


@pytest.mark.parametrize("rel,shrink", [
    ("dense/obj/uttt_dense_r2.yaml", dict(attn_head_dim=16, fw_head_dim=16)),
    ("ownership/obj/ttt_dense.yaml", dict(attn_head_dim=16, fw_head_dim=16)),
    ("reference/obj/gated_deltanet.yaml", dict(attn_head_dim=16, fw_num_heads=4)),
    ("transformer/obj/transformer.yaml", dict(attn_head_dim=16)),
], ids=["uttt-dense", "ttt-dense", "gated-deltanet", "transformer"])
def test_whole_model_matches_the_reference(rel, shrink, monkeypatch):
    """The reference's ``uttt_nvs.models.lvsm.Images2latent3D`` (rays, Plucker embedding, patch tokens, block stack,
    decoder, loss) against this package's model from the same YAML file, shrunk to 2 layers of width 64 on 32 x 32
    images: same state dict, same scenes, bf16 autocast.  ``torch.cross`` of a bf16 and an fp32 operand is promoted by
    the CUDA autocast rules but not by the CPU ones, so the test promotes it."""
    import copy
    import yaml
    _reference("transformer_block")
    from easydict import EasyDict
    from uttt_nvs.models.lvsm import Images2latent3D
    from uttt_b200.nvs.data import SyntheticScenes
    from uttt_b200.nvs.model import LVSMModel
    cross = torch.cross
    monkeypatch.setattr(torch, "cross", lambda a, b, dim=-1: cross(a.float(), b.float(), dim=dim))
    with open(os.path.join(REF, "uttt_nvs", "configs", rel)) as fh:
        cfg = yaml.safe_load(fh)
    cfg["model"].update(dim=64, layers=2, image_size=32)
    cfg["model"]["block_config"]["params"].update(shrink)
    cfg["training"].update(num_views=4, lpips_loss_weight=0.0, perceptual_loss_weight=0.0)
    torch.manual_seed(0)
    ref = Images2latent3D(EasyDict(copy.deepcopy(cfg)))
    ours = LVSMModel(copy.deepcopy(cfg))
    res = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    batch = next(SyntheticScenes(2, 4, 32, seed=3, rank=0, pin=False))
    with torch.autocast("cpu", dtype=torch.bfloat16):
        out_r = ref({k: v.clone() for k, v in batch.items()})
        out_o = ours({k: v.clone() for k, v in batch.items()})
    loss_r, loss_o = out_r["loss_metrics"]["loss"], out_o["loss_metrics"]["loss"]
    assert abs(float(loss_o) - float(loss_r)) < 2e-3 * abs(float(loss_r))
    assert out_o["rendering"].shape == out_r["rendering"].shape == (2, 3, 3, 32, 32)
    assert (out_o["rendering"].float() - out_r["rendering"].float()).abs().mean() < 3e-3
    torch.testing.assert_close(out_o["loss_metrics"]["psnr_loc"].float(), out_r["loss_metrics"]["psnr_loc"].float(),
                               atol=2e-2, rtol=0)
    torch.testing.assert_close(out_o["target"]["image"], out_r["target"]["image"])
    torch.testing.assert_close(out_o["input"]["c2w"], out_r["input"]["c2w"])
    loss_r.backward()
    loss_o.backward()
    g_r = ref.image_tokenizer[1].weight.grad.flatten().float()
    g_o = ours.image_tokenizer[1].weight.grad.flatten().float()
    assert torch.nn.functional.cosine_similarity(g_o, g_r, dim=0) > 0.99
    g_r = ref.image_token_decoder[1].weight.grad.flatten().float()
    g_o = ours.image_token_decoder[1].weight.grad.flatten().float()
    assert torch.nn.functional.cosine_similarity(g_o, g_r, dim=0) > 0.999


def _synthetic_matconvnet_vgg19(path, seed=0):
    """A file in the layout of ``imagenet-vgg-verydeep-19.mat`` with random filters: ``layers`` is a 1 x 37 cell of
    1 x 1 structs (name, type, weights), ``weights`` a 1 x 2 cell (filters [h, w, in, out], bias)."""
    import numpy as np
    import scipy.io
    rng = np.random.default_rng(seed)
    channels = [64, 64, 128, 128, 256, 256, 256, 256, 512, 512, 512, 512, 512, 512, 512, 512]
    conv_at = (0, 2, 5, 7, 10, 12, 14, 16, 19, 21, 23, 25, 28, 30, 32, 34)
    layers = np.empty((1, 37), dtype=object)
    c_in, k = 3, 0
    for i in range(37):
        if i in conv_at:
            c_out = channels[k]
            cell = np.empty((1, 2), dtype=object)
            cell[0, 0] = (rng.standard_normal((3, 3, c_in, c_out)) * (2.0 / (9 * c_in)) ** 0.5).astype(np.float32)
            cell[0, 1] = (rng.standard_normal((c_out, 1)) * 0.1).astype(np.float32)
            layers[0, i] = {"name": f"conv{k}", "type": "conv", "weights": cell}
            c_in, k = c_out, k + 1
        else:
            layers[0, i] = {"name": f"other{i}", "type": "relu", "weights": np.empty((1, 0), dtype=object)}
    scipy.io.savemat(path, {"layers": layers})


def test_perceptual_loss_matches_the_reference(tmp_path, monkeypatch):
    """The VGG-19 perceptual loss against the reference's module, both reading the same MatConvNet-layout file
    (random filters: the real file cannot be downloaded here): value and gradient with respect to the prediction."""
    _reference("ttt_dense_block")
    mat = str(tmp_path / "imagenet-vgg-verydeep-19.mat")
    _synthetic_matconvnet_vgg19(mat)
    monkeypatch.setenv("VGG19_MAT_PATH", mat)
    from uttt_nvs.models.perceptual_loss import PerceptualLoss as Theirs
    from uttt_b200.nvs.perceptual import PerceptualLoss as Ours
    theirs, ours = Theirs(), Ours()
    assert not list(p for p in ours.parameters() if p.requires_grad)
    torch.manual_seed(0)
    pred = torch.rand(2, 3, 64, 64)
    target = torch.rand(2, 3, 64, 64)
    pr, po = pred.clone().requires_grad_(), pred.clone().requires_grad_()
    lr_, lo = theirs(pr, target), ours(po, target)
    torch.testing.assert_close(lo, lr_, rtol=1e-5, atol=1e-6)
    lr_.backward()
    lo.backward()
    torch.testing.assert_close(po.grad, pr.grad, rtol=1e-4, atol=1e-7)
    assert float(ours(target, target)) == 0.0
