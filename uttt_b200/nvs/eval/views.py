"""Frozen view manifests and the fixed-view dataset (uttt_nvs/eval/build_view_manifest.py, fixed_view_dataset.py).

A view manifest freezes, for every scene of a dataset manifest, an ordered list of ``num_views`` frame indices
drawn with a per-scene generator seeded from (seed, scene id).  View 0 conditions, views 1.. are scored.

    python -m uttt_b200.nvs.eval.views --manifest scenes.txt --output views.json [--num-views 24] [--seed 9595]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
from typing import Dict, List

import torch
from torch.utils.data import Dataset

from ..data import NVSDataset


def scene_id(path: str) -> str:
    base = os.path.basename(path)
    stem = base[:-5] if base.endswith(".json") else base
    parent = os.path.basename(os.path.dirname(path))
    return f"{parent}/{stem}" if parent else stem


def _scene_seed(seed: int, sid: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{sid}".encode()).digest()[:8], "little")


def build_view_manifest(manifest: str, num_views: int = 24, seed: int = 9595, strict: bool = True) -> Dict:
    with open(manifest) as fh:
        scenes = [ln.strip() for ln in fh if ln.strip()]
    entries, skipped = [], []
    for path in scenes:
        with open(path) as fh:
            n_frames = len(json.load(fh)["frames"])
        sid = scene_id(path)
        if n_frames < num_views:
            if strict:
                raise ValueError(f"scene {sid} has {n_frames} frames, {num_views} are needed")
            skipped.append(sid)
            continue
        g = torch.Generator().manual_seed(_scene_seed(seed, sid) % (2 ** 63))
        picks = torch.randperm(n_frames, generator=g)[:num_views].tolist()
        entries.append({"scene_id": sid, "path": path, "frames": picks})
    digest = hashlib.sha256(json.dumps(entries, sort_keys=True).encode()).hexdigest()
    return {"version": 1, "num_views": num_views, "seed": seed, "source_manifest": os.path.abspath(manifest),
            "scenes": entries, "skipped": skipped, "sha256": digest}


def load_view_manifest(path: str) -> Dict:
    with open(path) as fh:
        doc = json.load(fh)
    digest = hashlib.sha256(json.dumps(doc["scenes"], sort_keys=True).encode()).hexdigest()
    if doc.get("sha256") and doc["sha256"] != digest:
        raise ValueError(f"view manifest {path} was edited after it was frozen (checksum mismatch)")
    return doc


class FixedViewDataset(Dataset):
    """Scenes of a frozen view manifest, each returned with exactly its frozen, ordered views."""

    def __init__(self, view_manifest: str, image_size: int, shard_index: int = 0, num_shards: int = 1,
                 max_scenes: int = 0):
        doc = load_view_manifest(view_manifest)
        scenes: List[Dict] = doc["scenes"]
        if max_scenes:
            scenes = scenes[:max_scenes]
        self.scenes = scenes[shard_index::num_shards]
        self.num_views = doc["num_views"]
        self._loader = NVSDataset.__new__(NVSDataset)
        self._loader.image_size = image_size

    def __len__(self):
        return len(self.scenes)

    def __getitem__(self, idx: int):
        entry = self.scenes[idx]
        with open(entry["path"]) as fh:
            frames = json.load(fh)["frames"]
        imgs, intr, poses = zip(*[self._loader._load_frame(frames[i]) for i in entry["frames"]])
        return {"image": torch.stack(imgs), "fxfycxcy": torch.stack(intr), "c2w": torch.stack(poses),
                "scene_id": entry["scene_id"]}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--manifest", required=True)
    ap.add_argument("--output", required=True, help="Output JSON path.")
    ap.add_argument("--num-views", type=int, default=24)
    ap.add_argument("--seed", type=int, default=9595)
    ap.add_argument("--allow-short-scenes", action="store_true")
    args = ap.parse_args(argv)
    doc = build_view_manifest(args.manifest, args.num_views, args.seed, strict=not args.allow_short_scenes)
    tmp = args.output + ".tmp"
    with open(tmp, "w") as fh:
        json.dump(doc, fh, indent=1)
    os.replace(tmp, args.output)
    print(f"froze {len(doc['scenes'])} scenes x {args.num_views} views -> {args.output}")


if __name__ == "__main__":
    main()
