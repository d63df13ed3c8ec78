"""Full-test evaluation of view-synthesis checkpoints: registry, frozen view manifests, per-view metrics,
scene-bootstrap confidence intervals, shard merge, runtime fingerprint and comparison grids.

Behavioural reference: uttt_nvs/eval/{evaluate,common,fixed_view_dataset,build_view_manifest,aggregate,
merge_sharded_evaluations,runtime_fingerprint,render_comparison,statistics,metrics}.py.
"""
from .registry import Experiment, load_registry, preflight
from .views import FixedViewDataset, build_view_manifest, load_view_manifest
