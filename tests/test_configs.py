import glob
import os

from uttt_b200.config import load_config
from uttt_b200.tools.check_configs import ROOT, catalog, check_all


def test_every_shipped_config_validates():
    n, errs = check_all()
    assert n >= 100 and not errs, errs[:5]


def test_catalog_is_fresh():
    assert open(os.path.join(ROOT, "CATALOG.md")).read() == catalog()


def test_architecture_json_schema_accepts_upstream_style_keys():
    """Unknown keys are preserved and model_type aliases resolve (schema compatibility)."""
    path = glob.glob(os.path.join(ROOT, "lm", "main", "760M", "uttt_moe.json"))[0]
    cfg = load_config(path, attention_bias=False, transformers_version="5.5.0")
    assert cfg.extra["transformers_version"] == "5.5.0" and cfg.memory_num_experts == 96


def _nvs_errors(tmp_path, mutate):
    import copy
    import yaml
    from uttt_b200.tools.check_configs import check_nvs_yaml
    cfg = copy.deepcopy(yaml.safe_load(open(os.path.join(ROOT, "nvs", "ownership", "obj", "uttt_moe_e64a1.yaml"))))
    mutate(cfg)
    path = tmp_path / "probe.yaml"
    path.write_text(yaml.safe_dump(cfg))
    return check_nvs_yaml(str(path))


def test_checker_rejects_broken_view_synthesis_files(tmp_path):
    """The invalid cases of tests/test_configs.py:23-43 of the reference are all reported, none raises."""
    assert not _nvs_errors(tmp_path, lambda c: None)
    for key, value in (("num_experts", 0), ("num_active_experts", 65), ("pool_mode", "per_block"), ("fw_head_dim", 31)):
        assert _nvs_errors(tmp_path, lambda c: c["model"]["block_config"]["params"].__setitem__(key, value)), key
    for key, value in (("total_batch_size", 127), ("grad_accum_steps", 0), ("num_views", True),
                       ("batch_size_per_gpu", -1)):
        assert _nvs_errors(tmp_path, lambda c: c["training"].__setitem__(key, value)), key
    errs = _nvs_errors(tmp_path, lambda c: c["model"].__setitem__("class_name", "uttt_nvs.models.lvsm.DoesNotExist"))
    assert errs and "not defined" in errs[0]
    assert not _nvs_errors(tmp_path, lambda c: c["model"].__setitem__("class_name",
                                                                      "uttt_nvs.models.lvsm_moe.Images2latent3D"))


def test_checker_rejects_broken_language_model_files(tmp_path):
    import json
    from uttt_b200.tools.check_configs import check_lm_json
    base = json.load(open(os.path.join(ROOT, "lm", "main", "124M", "uttt_moe.json")))
    for updates in ({"model_type": "made_up"}, {"num_heads": 11}, {"memory_num_active_experts": 49},
                    {"memory_pool_mode": "per_block"}, {"chunk_size": 0}):
        path = tmp_path / "probe.json"
        path.write_text(json.dumps({**base, **updates}))
        assert check_lm_json(str(path)), updates
