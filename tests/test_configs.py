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
