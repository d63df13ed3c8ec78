"""Full-test evaluation pipeline on a toy dataset: frozen view manifests, registry preflight, sharded scoring,
shard merge, aggregate tables, comparison grids, runtime fingerprint, perceptual modules."""
import json
import os

import pytest
import torch
import yaml

from uttt_b200.nvs.data import make_toy_dataset
from uttt_b200.nvs.eval import aggregate as agg
from uttt_b200.nvs.eval import evaluate as ev
from uttt_b200.nvs.eval import merge_shards, render_comparison
from uttt_b200.nvs.eval.fingerprint import runtime_fingerprint
from uttt_b200.nvs.eval.registry import load_registry, preflight
from uttt_b200.nvs.eval.views import FixedViewDataset, build_view_manifest, load_view_manifest
from uttt_b200.nvs.eval.views import main as views_main


def _model_cfg():
    p = dict(attn_head_dim=32, fw_head_dim=32, inter_multi=2, fw_inter_multi=1, use_muon=False, num_experts=4,
             num_active_experts=2, l2_norm=True, pool_mode="shared", router_share_mode="share_all",
             aggregate_write=True, load_balancing_loss_alpha=1e-5)
    return {"exp_name": "t", "model": {"image_size": 32, "patch_size": 8, "dim": 64, "layers": 2,
                                       "block_config": {"type": "uttt_nvs.models.uttt_moe_block.MemoryModel",
                                                        "params": p}},
            "training": {"num_views": 6}}


@pytest.fixture()
def toy(tmp_path):
    manifest = make_toy_dataset(str(tmp_path / "data"), num_scenes=4, num_frames=10, image_size=32, seed=3)
    views = str(tmp_path / "views.json")
    views_main(["--dataset-manifest", manifest, "--dataset", "toy", "--output", views, "--num-views", "6",
                "--seed", "9595"])
    cfg = tmp_path / "model.yaml"
    cfg.write_text(yaml.safe_dump(_model_cfg()))
    reg = tmp_path / "experiments.yaml"
    reg.write_text(yaml.safe_dump({
        "defaults": {"checkpoint_root": str(tmp_path / "ckpts"), "output_root": str(tmp_path / "out"), "num_views": 6},
        "datasets": {"toy": {"manifest": manifest, "view_manifest": views, "image_size": 32, "num_scenes": 4}},
        "experiments": [
            {"name": "toy/a", "dataset": "toy", "config": str(cfg), "checkpoint": "a.pt", "paper_model": "A"},
            {"name": "toy/b", "dataset": "toy", "config": str(cfg), "checkpoint": "b.pt", "display_name": "B"}]}))
    return {"manifest": manifest, "views": views, "registry": reg, "root": tmp_path}


def test_view_manifest_is_frozen_and_deterministic(toy):
    a = build_view_manifest(toy["manifest"], 6, 9595)
    b = build_view_manifest(toy["manifest"], 6, 9595)
    c = build_view_manifest(toy["manifest"], 6, 1)
    assert a["scenes"] == b["scenes"] and a["scenes"] != c["scenes"]
    assert all(len(set(s["frame_indices"])) == 6 for s in a["scenes"])
    doc = load_view_manifest(toy["views"])
    doc["scenes"][0]["frame_indices"] = doc["scenes"][0]["frame_indices"][::-1]
    edited = toy["root"] / "edited.json"
    edited.write_text(json.dumps(doc))
    with pytest.raises(ValueError):
        load_view_manifest(str(edited))
    with pytest.raises(ValueError):
        build_view_manifest(toy["manifest"], 24, 9595)          # scenes have only 10 frames
    ds = FixedViewDataset(toy["views"], 32, shard_index=1, num_shards=2)
    assert len(ds) == 2 and ds[0]["image"].shape == (6, 3, 32, 32)


def test_preflight_refuses_missing_inputs(toy):
    reg = load_registry(toy["registry"])
    exp = reg["toy/a"]
    assert exp.scored_views == 5
    problems = preflight(exp)
    assert len(problems) == 1 and "checkpoint not found" in problems[0]
    os.remove(toy["views"])
    assert any("view manifest" in p for p in preflight(exp, require_checkpoint=False))
    with pytest.raises(SystemExit):
        ev.main(["--registry", str(toy["registry"]), "--experiment", "toy/a", "--device", "cpu"])


def test_sharded_evaluation_merge_aggregate_and_grids(toy):
    reg_path = str(toy["registry"])
    shards = toy["root"] / "shards"
    for name in ("toy/a", "toy/b"):
        for i in range(2):
            ev.main(["--registry", reg_path, "--experiment", name, "--output-root", str(shards), "--shard-index", str(i),
                     "--num-shards", "2", "--device", "cpu", "--amp-dtype", "fp32", "--bootstrap-samples", "200",
                     "--allow-missing-checkpoint"])
    with pytest.raises(SystemExit):                      # finished shards are not silently overwritten
        ev.main(["--registry", reg_path, "--experiment", "toy/a", "--output-root", str(shards), "--shard-index", "0",
                 "--num-shards", "2", "--device", "cpu", "--allow-missing-checkpoint"])
    reg = load_registry(reg_path)
    out = toy["root"] / "out"
    for name in ("toy/a", "toy/b"):
        s = merge_shards.merge(reg[name], shards, 2, out, bootstrap_samples=200)
        assert s["num_scenes"] == 4 and s["num_rows"] == 4 * 5
        assert s["psnr"]["ci95"][0] <= s["psnr"]["mean"] <= s["psnr"]["ci95"][1]
    with pytest.raises(FileNotFoundError):
        merge_shards.merge(reg["toy/a"], shards, 3, toy["root"] / "other")
    tables = agg.aggregate(reg_path, out)
    assert len(tables["toy"]) == 2 and (out / "aggregate_toy.md").read_text().count("\n") == 4
    meta = json.loads((ev.shard_dir(shards, "toy/a", 0, 2) / "run_metadata.json").read_text())
    assert meta["fingerprint"]["torch"] == torch.__version__ and meta["registry_entry"]["paper_model"] == "A"
    files = render_comparison.render(reg_path, "toy", ["toy/a", "toy/b"], toy["root"] / "grids", scene_count=2,
                                     view_indices=(1, 3, 5), device="cpu", amp_dtype="fp32",
                                     allow_missing_checkpoint=True)
    assert len(files) == 2 and all(os.path.getsize(f) > 0 for f in files)
    from PIL import Image
    w, h = Image.open(files[0]).size
    assert (w, h) == (3 * 34 + 2, 3 * 34 + 2)


def test_fingerprint_and_perceptual_modules():
    fp = runtime_fingerprint()
    assert {"python", "torch", "git_commit", "native_kernels"} <= set(fp)
    from uttt_b200.nvs.perceptual import LPIPSVGG, PerceptualLoss
    with pytest.raises(FileNotFoundError):
        PerceptualLoss()
    loss = PerceptualLoss(allow_random=True)
    a = torch.rand(2, 3, 32, 32, requires_grad=True)
    b = torch.rand(2, 3, 32, 32)
    val = loss(a, b)
    val.backward()
    assert val.item() > 0 and a.grad.abs().sum() > 0 and float(loss(b, b)) == 0.0
    d = LPIPSVGG(allow_random=True)
    assert d(b, b).abs().max() == 0 and d(a.detach(), b).shape == (2,)
