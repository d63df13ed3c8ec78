"""Full-test evaluation pipeline on a toy dataset: frozen view manifests, registry preflight, sharded scoring,
shard merge, aggregate tables, comparison grids, runtime fingerprint, perceptual modules."""
import json
import os

import numpy as np
import pytest
import torch
import yaml

from uttt_b200.nvs.data import make_toy_dataset
from uttt_b200.nvs.eval import aggregate as agg
from uttt_b200.nvs.eval import evaluate as ev
from uttt_b200.nvs.eval import merge_shards, render_comparison
from uttt_b200.nvs.eval import stats
from uttt_b200.nvs.eval.fingerprint import (canonical_json_sha256, deterministic_runtime_fingerprint,
                                            evaluation_code_sha256, file_sha256, runtime_fingerprint,
                                            runtime_fingerprint_sha256, validate_runtime_fingerprint)
from uttt_b200.nvs.eval.registry import experiment_dir, load_registry, preflight, select_experiments, validate_v_gap
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
    reg.write_text(yaml.safe_dump({                              # the reference's registry layout
        "version": 1,
        "defaults": {"checkpoint_root": str(tmp_path / "ckpts"), "output_root": str(tmp_path / "out"), "num_views": 6,
                     "seed": 9595},
        "datasets": [{"id": "toy", "display_name": "Toy", "local_manifest": manifest, "view_manifest": views,
                      "expected_scenes": 4, "expected_rows": 20}],
        "experiments": [
            {"id": "toy_a", "dataset": "toy", "model": "a", "paper_model": "A", "config": str(cfg),
             "checkpoint": "a/checkpoint.pt", "checkpoint_step": 10, "checkpoint_impl": "uttt_moe", "group": "g",
             "display_name": "A-small"},
            {"id": "toy_b", "dataset": "toy", "model": "b", "paper_model": "B", "config": str(cfg),
             "checkpoint": "b/checkpoint.pt", "checkpoint_step": 10, "checkpoint_impl": "uttt_moe", "group": "g",
             "display_name": "B-small"}]}))
    return {"manifest": manifest, "views": views, "registry": reg, "root": tmp_path, "config": cfg}


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
    assert [s["scene_index"] for s in ds.scenes] == [1, 3]      # strided shard
    assert len(FixedViewDataset(toy["views"], 32, shard_index=1, num_shards=2, max_scenes=1)) == 1


def test_registry_layouts_and_preflight(toy):
    reg = load_registry(toy["registry"])
    exp = reg["toy_a"]
    assert exp.id == "toy_a" and exp.scored_views == 5 and exp.expected_rows == 20 and exp.display_name == "A-small"
    assert exp.checkpoint == toy["root"] / "ckpts" / "a" / "checkpoint.pt" and exp.image_size is None
    assert experiment_dir(toy["root"] / "out", exp) == toy["root"] / "out" / "toy" / "toy_a"
    assert select_experiments(toy["registry"], ["toy"]) == ["toy_a", "toy_b"]
    assert select_experiments(toy["registry"], ["other"]) == []
    problems = preflight(exp)
    assert len(problems) == 1 and "checkpoint not found" in problems[0]
    # mapping form with the older key names, and a reference-style config path
    doc = yaml.safe_load(toy["registry"].read_text())
    doc["datasets"] = {"toy": {"manifest": toy["manifest"], "view_manifest": toy["views"], "num_scenes": 4,
                               "image_size": 32}}
    doc["experiments"] = [{"name": "toy/x", "dataset": "toy", "checkpoint": "x.pt",
                           "config": "uttt_nvs/configs/ownership/obj/uttt_moe_e64a1.yaml"}]
    older = toy["root"] / "older.yaml"
    older.write_text(yaml.safe_dump(doc))
    x = load_registry(older)["toy/x"]
    assert x.expected_rows == 20 and x.image_size == 32 and x.config.is_file()
    assert x.config.parts[-5:] == ("configs", "nvs", "ownership", "obj", "uttt_moe_e64a1.yaml")
    for breakage, error in ((lambda d: d.pop("defaults"), ValueError),
                            (lambda d: d.update(experiments={}), ValueError),
                            (lambda d: d["experiments"].append(dict(d["experiments"][0])), ValueError),
                            (lambda d: d["experiments"][0].update(dataset="nope"), KeyError)):
        bad = yaml.safe_load(toy["registry"].read_text())
        breakage(bad)
        (toy["root"] / "bad.yaml").write_text(yaml.safe_dump(bad))
        with pytest.raises(error):
            load_registry(toy["root"] / "bad.yaml")
    os.remove(toy["views"])
    assert any("view manifest" in p for p in preflight(exp, require_checkpoint=False))
    with pytest.raises(SystemExit):
        ev.main(["--registry", str(toy["registry"]), "--experiment", "toy_a", "--device", "cpu"])


def test_attention_gap_must_be_declared(toy):
    exp = load_registry(toy["registry"])["toy_a"]
    cfg = _model_cfg()
    assert validate_v_gap(exp, cfg) is None
    cfg["model"]["block_config"]["params"]["v_gap"] = 4
    with pytest.raises(ValueError, match="expected v_gap=None"):
        validate_v_gap(exp, cfg)
    exp.raw["expected_v_gap"] = 4
    with pytest.raises(ValueError, match="allow_nonnull_v_gap"):
        validate_v_gap(exp, cfg)
    exp.raw["allow_nonnull_v_gap"] = True
    assert validate_v_gap(exp, cfg) == 4


def test_bootstrap_summaries_follow_the_published_protocol():
    """The intervals restated with numpy alone: default_rng(seed), integer draws in chunks of 512 resamples, seed
    offsets of 100000 per metric and 1 per view; scene-macro means."""
    rng = np.random.default_rng(0)
    rows = [{"dataset": "d", "model": "m", "scene_id": f"s{s:02d}", "view_index": v,
             "psnr": float(20 + rng.normal()), "ssim": float(0.8 + 0.01 * rng.normal()),
             "lpips": float("nan") if s == 3 else float(0.2 + 0.01 * rng.normal())}
            for s in range(7) for v in range(1, 4)]
    overall, per_view = stats.summarize_records(rows, bootstrap_samples=700, bootstrap_seed=9595, scored_views=3)
    assert overall["num_valid_scenes"] == 7 and overall["num_valid_samples"] == 21
    assert overall["overall_lpips_n_valid"] == 6 and overall["overall_psnr_n_valid"] == 7

    def interval(values, seed, samples=700):
        x, g, means = np.asarray(values), np.random.default_rng(seed), []
        for lo in range(0, samples, 512):
            n = min(512, samples - lo)
            means.append(x[g.integers(0, x.size, size=(n, x.size))].mean(axis=1))
        return np.quantile(np.concatenate(means), [0.025, 0.975])

    scene_psnr = [np.mean([r["psnr"] for r in rows if r["scene_id"] == f"s{s:02d}"]) for s in range(7)]
    assert overall["overall_psnr"] == pytest.approx(np.mean(scene_psnr))
    lo, hi = interval(scene_psnr, 9595)
    assert (overall["overall_psnr_ci95_low"], overall["overall_psnr_ci95_high"]) == (pytest.approx(lo), pytest.approx(hi))
    scene_lpips = [np.mean([r["lpips"] for r in rows if r["scene_id"] == f"s{s:02d}"]) for s in range(7) if s != 3]
    lo, hi = interval(scene_lpips, 9595 + 200_000)
    assert overall["overall_lpips_ci95_low"] == pytest.approx(lo) and overall["overall_lpips_ci95_high"] == pytest.approx(hi)
    row = next(r for r in per_view if r["metric"] == "ssim" and r["view_index"] == 2)
    vals = [r["ssim"] for r in rows if r["view_index"] == 2]
    lo, hi = interval(vals, 9595 + 100_000 + 2)
    assert row["n_valid"] == 7 and row["mean"] == pytest.approx(np.mean(vals))
    assert row["ci95_low"] == pytest.approx(lo) and row["ci95_high"] == pytest.approx(hi)
    assert len(per_view) == 9 and list(per_view[0]) == list(stats.PER_VIEW_FIELDS)
    assert stats.bootstrap_mean_ci([], 10, 0) == (None, None) and stats.bootstrap_mean_ci([2.0], 10, 0) == (2.0, 2.0)
    with pytest.raises(ValueError, match="view_index"):
        stats.summarize_records([dict(rows[0], view_index=4)], scored_views=3)
    with pytest.raises(ValueError, match="one dataset and one model"):
        stats.summarize_records(rows + [dict(rows[0], model="other")], scored_views=3)
    with pytest.raises(ValueError, match="missing columns"):
        stats.clean_records([{"dataset": "d"}])
    with pytest.raises(RuntimeError, match="incomplete"):
        stats.validate_complete(rows[:-1], 7, 20, 3)
    with pytest.raises(RuntimeError, match="expected 8 scenes"):
        stats.validate_complete(rows, 8, 24, 3)


def test_sharded_evaluation_merge_aggregate_and_grids(toy):
    reg_path = str(toy["registry"])
    shards = toy["root"] / "shards"
    for name in ("toy_a", "toy_b"):
        for i in range(2):
            assert ev.main(["--registry", reg_path, "--experiment", name, "--output-root", str(shards / f"shard_{i}"),
                            "--shard-index", str(i), "--num-shards", "2", "--device", "cpu", "--amp-dtype", "fp32",
                            "--bootstrap-samples", "200", "--allow-missing-checkpoint"]) == 0
    with pytest.raises(SystemExit):                      # finished shards are not silently overwritten
        ev.main(["--registry", reg_path, "--experiment", "toy_a", "--output-root", str(shards / "shard_0"),
                 "--shard-index", "0", "--num-shards", "2", "--device", "cpu", "--allow-missing-checkpoint"])
    d = shards / "shard_0" / "toy" / "toy_a"
    assert {p.name for p in d.iterdir()} >= {"raw_metrics.csv", "per_view_summary.csv", "overall_summary.json",
                                              "run_metadata.json", "completion.json"}
    assert not (d / "raw_metrics.partial.csv").exists()
    header, first = (d / "raw_metrics.csv").read_text().splitlines()[:2]
    assert header == "dataset,model,scene_id,view_index,psnr,ssim,lpips"
    assert first.startswith("toy,A-small,scene_000,1,") and first.endswith(",")          # no LPIPS weights here
    meta = json.loads((d / "run_metadata.json").read_text())
    assert meta["protocol_version"] == "nvs-eval-v2" and meta["shard_index"] == 0 and meta["num_shards"] == 2
    assert meta["runtime"]["torch"] == torch.__version__ and meta["paper_model"] == "A" and meta["v_gap"] is None
    assert meta["config_sha256"] == file_sha256(toy["config"]) and meta["conditioning_protocol"] == "teacher_forced_sequential"
    done = json.loads((d / "completion.json").read_text())
    assert done["state"] == "complete" and done["expected_rows"] == 10
    assert done["raw_metrics_sha256"] == file_sha256(d / "raw_metrics.csv") == done["artifact_sha256"]["raw_metrics.csv"]
    other = json.loads((shards / "shard_1" / "toy" / "toy_a" / "run_metadata.json").read_text())
    assert other["runtime_sha256"] == meta["runtime_sha256"]              # nothing shard- or host-specific in it

    reg = load_registry(reg_path)
    out = toy["root"] / "out"
    for name in ("toy_a", "toy_b"):
        s = merge_shards.merge(reg[name], shards, 2, out, bootstrap_samples=200)
        assert s["num_valid_scenes"] == 4 and s["num_valid_samples"] == 20 and s["expected_rows"] == 20
        assert s["overall_psnr_ci95_low"] <= s["overall_psnr"] <= s["overall_psnr_ci95_high"]
        assert s["overall_lpips"] is None and s["overall_lpips_n_valid"] == 0
    merged = json.loads((out / "toy" / "toy_a" / "run_metadata.json").read_text())
    assert merged["shard_index"] is None and merged["merge_protocol"] == "deterministic strided scene shards"
    with pytest.raises(FileExistsError):
        merge_shards.merge(reg["toy_a"], shards, 2, out)
    with pytest.raises(ValueError, match="num_shards"):
        merge_shards.merge(reg["toy_a"], shards, 3, toy["root"] / "other")
    (shards / "shard_1" / "toy" / "toy_b" / "completion.json").unlink()
    with pytest.raises(FileNotFoundError, match="incomplete shard 1"):
        merge_shards.merge(reg["toy_b"], shards, 2, toy["root"] / "other")

    # one unsharded run gives the same table as the merge of its shards
    assert ev.main(["--registry", reg_path, "--experiment", "toy_a", "--output-root", str(toy["root"] / "single"),
                    "--device", "cpu", "--amp-dtype", "fp32", "--bootstrap-samples", "200",
                    "--allow-missing-checkpoint"]) == 0

    def table(path):
        return sorted(stats.read_raw_csv(path), key=lambda r: (r["scene_id"], r["view_index"]))

    a, b = table(toy["root"] / "single" / "toy" / "toy_a" / "raw_metrics.csv"), table(out / "toy" / "toy_a" / "raw_metrics.csv")
    assert [(r["scene_id"], r["view_index"]) for r in a] == [(r["scene_id"], r["view_index"]) for r in b]

    info = agg.aggregate(reg_path, out)
    assert info["runs"] == 2 and info["raw_rows"] == 40 and info["per_view_rows"] == 2 * 3 * 5 and info["missing"] == 0
    rows = stats.read_csv(out / "aggregate" / "all_overall_metrics.csv")
    assert [r["experiment_id"] for r in rows] == ["toy_a", "toy_b"] and rows[0]["checkpoint_impl"] == "uttt_moe"
    assert (out / "aggregate" / "table_toy.md").read_text().count("\n") == 4
    assert json.loads((out / "aggregate" / "missing_runs.json").read_text()) == []
    with pytest.raises(FileNotFoundError):
        agg.aggregate(reg_path, toy["root"] / "single")                 # toy_b was not run there
    assert agg.aggregate(reg_path, toy["root"] / "single", allow_incomplete=True)["missing"] == 1

    files = render_comparison.render(reg_path, "toy", ["toy_a", "toy_b"], toy["root"] / "grids", scene_count=2,
                                     view_indices=(1, 3, 5), device="cpu", amp_dtype="fp32",
                                     allow_missing_checkpoint=True)
    assert len(files) == 2 and all(os.path.getsize(f) > 0 for f in files)
    from PIL import Image
    assert Image.open(files[0]).size == (32 * 4, render_comparison.HEADER + (32 + render_comparison.CAPTION) * 3)
    index = json.loads((toy["root"] / "grids" / "toy" / "index.json").read_text())
    assert index["view_indices"] == [1, 3, 5] and index["models"] == ["A-small", "B-small"]
    assert len(index["scene_ids"]) == 2 and index["files"] == files
    folder = os.path.dirname(files[0])
    assert os.path.basename(folder) == render_comparison.safe_name(index["scene_ids"][0])
    names = set(os.listdir(folder))
    assert {"input_view_00.png", "comparison.png", "ground_truth_view_01.png", "ground_truth_view_05.png",
            "A-small_view_01.png", "B-small_view_03.png"} <= names and len(names) == 2 + 3 * 3
    per_view = index["metrics"]["A-small"][index["scene_ids"][0]]["3"]
    assert set(per_view) == {"psnr", "ssim", "lpips"} and per_view["psnr"] > 0
    named = render_comparison.render(reg_path, "toy", ["toy_a"], toy["root"] / "grids_named",
                                     scene_ids=[index["scene_ids"][1]], view_indices=(2,), device="cpu",
                                     amp_dtype="fp32", allow_missing_checkpoint=True)
    assert len(named) == 1 and render_comparison.safe_name(index["scene_ids"][1]) in named[0]
    with pytest.raises(KeyError):
        render_comparison.render(reg_path, "toy", ["toy_a"], toy["root"] / "grids_named", scene_ids=["nope"],
                                 device="cpu", amp_dtype="fp32", allow_missing_checkpoint=True)


def test_smoke_runs_stay_out_of_the_full_results(toy):
    assert ev.main(["--registry", str(toy["registry"]), "--experiment", "toy_b", "--max-scenes", "2", "--device", "cpu",
                    "--amp-dtype", "fp32", "--bootstrap-samples", "50", "--allow-missing-checkpoint"]) == 0
    d = toy["root"] / "eval_outputs_smoke" / "n2" / "toy" / "toy_b"
    assert json.loads((d / "overall_summary.json").read_text())["num_valid_scenes"] == 2
    assert not (toy["root"] / "out" / "toy" / "toy_b").exists()


def test_strict_checkpoints(toy):
    exp = load_registry(toy["registry"])["toy_a"]
    model, _ = ev.load_model(exp, "cpu", allow_missing_checkpoint=True)
    exp.checkpoint.parent.mkdir(parents=True)
    sd = {"module._orig_mod." + k: v for k, v in model.state_dict().items()}
    torch.save({"model": sd, "fwdbwd_pass_step": 7, "param_update_step": 3}, exp.checkpoint)
    _, info = ev.load_model(exp, "cpu")
    assert info == {"fwdbwd_pass_step": 7, "param_update_step": 3}
    sd.pop(next(iter(sd)))
    torch.save({"model": sd}, exp.checkpoint)
    with pytest.raises(RuntimeError, match="Missing key"):
        ev.load_model(exp, "cpu")
    torch.save(sd, exp.checkpoint)
    with pytest.raises(ValueError, match="Unsupported checkpoint format"):
        ev.load_model(exp, "cpu")


def test_deterministic_fingerprint_has_no_host_identity():
    fp = deterministic_runtime_fingerprint("cpu")
    validate_runtime_fingerprint(fp, require_cuda=False)
    assert runtime_fingerprint_sha256(fp) == runtime_fingerprint_sha256(dict(reversed(list(fp.items()))))
    with pytest.raises(ValueError, match="lacks GPU model"):
        validate_runtime_fingerprint(fp, require_cuda=True)
    with pytest.raises(ValueError, match="forbidden"):
        validate_runtime_fingerprint(dict(fp, numeric_flags=dict(fp["numeric_flags"], hostname="x")), require_cuda=False)
    with pytest.raises(ValueError, match="fields changed"):
        validate_runtime_fingerprint({k: v for k, v in fp.items() if k != "numpy"}, require_cuda=False)
    assert len(evaluation_code_sha256()) == 64 and canonical_json_sha256({"b": 1, "a": 2}) == canonical_json_sha256({"a": 2, "b": 1})


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
    # the VGG-16 trunk with the lpips package's key names for the heads; a term of the training loss, so differentiable
    names = [k for k in d.vgg.features.state_dict() if k.endswith(".weight")]
    assert len(names) == 13 and not any(p.requires_grad for p in d.parameters())
    a.grad = None
    d(a, b).sum().backward()
    assert a.grad is not None and a.grad.abs().sum() > 0


def test_output_folder_fingerprint():
    import hashlib
    from uttt_b200.nvs.eval.fingerprint import (NATURAL_OUTPUT_IDENTITY_ASSET_KEYS,
                                                natural_output_source_fingerprint_sha256 as fp)
    assets = {k: f"{i:064x}" for i, k in enumerate(NATURAL_OUTPUT_IDENTITY_ASSET_KEYS)}
    base = dict(experiment_id="gso_x", protocol_version="nvs-eval-v2", run_signature="s" * 64, identity_assets=assets,
                runtime_sha256="r" * 64, scene_count=2, scene_file_sha256={"a.pt": "1" * 64, "b.pt": "2" * 64})
    digest = fp(**base)
    # the published canonical form: sorted keys, compact separators, UTF-8
    payload = {"experiment_id": "gso_x", "protocol_version": "nvs-eval-v2", "run_signature": "s" * 64,
               "runtime_sha256": "r" * 64, "identity_assets": assets, "scene_count": 2,
               "scene_file_sha256": base["scene_file_sha256"]}
    want = hashlib.sha256(json.dumps(payload, ensure_ascii=False, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    assert digest == want and fp(**{**base, "scene_file_sha256": {"b.pt": "2" * 64, "a.pt": "1" * 64}}) == digest
    assert fp(**{**base, "experiment_id": "gso_y"}) != digest
    for broken in (dict(experiment_id=""), dict(scene_count=3), dict(scene_count=True),
                   dict(identity_assets={**assets, "extra": "x"}), dict(identity_assets={**assets, "code_commit": ""}),
                   dict(scene_file_sha256={"dir/a.pt": "1" * 64, "b.pt": "2" * 64})):
        with pytest.raises(ValueError):
            fp(**{**base, **broken})
