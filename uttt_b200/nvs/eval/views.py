"""Frozen view manifests and the fixed-view dataset (uttt_nvs/eval/build_view_manifest.py, fixed_view_dataset.py).

A view manifest freezes, for every scene of a local dataset manifest, an ordered list of ``num_views`` frame
indices, so that every checkpoint is scored on the same inputs and targets.  View 0 conditions, views 1.. are
scored.  The file layout and the selection rule are the reference's, so a manifest frozen by either
implementation selects the same frames and loads in both:

* ``schema_version 1``; top-level ``dataset, seed, num_views, selection_method, source_manifest,
  source_manifest_sha256, view_semantics {input: 0, targets: [1..]}, scenes``;
* per scene ``scene_index, scene_id, camera_path, camera_sha256, frame_indices, frame_ids``;
* selection: ``random.Random(s).sample(range(n_frames), num_views)`` with ``s`` = the first eight bytes
  (big-endian) of ``sha256(f"{seed}\\0{scene_id}")``: independent of the order of the dataset manifest.

This module adds ``selection_sha256`` (a digest of the ``scenes`` list; checked when present), which catches a
hand edit at load time instead of at the first read of the scene.

    python -m uttt_b200.nvs.eval.views --dataset-manifest scenes.txt --dataset gso --output views.json
        [--num-views 24] [--seed 9595] [--force]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import random
from typing import Dict, List, Optional

from torch.utils.data import Dataset

from ..data import NVSDataset

SCHEMA_VERSION = 1
DEFAULT_NUM_VIEWS = 24
DEFAULT_VIEW_SEED = 9595
SELECTION_METHOD = "per_scene_seeded_sample"
_GENERIC_STEMS = {"camera", "cameras", "metadata", "transforms", "transforms_train", "transforms_test"}


class ViewManifestError(ValueError):
    """A dataset manifest or a frozen view manifest is not usable for evaluation."""


def _local(path, what: str) -> str:
    path = str(path)
    if "://" in path:
        raise ViewManifestError(f"{what} must be local for reproducible evaluation, got {path!r}")
    return os.path.realpath(os.path.expanduser(path))


def read_local_manifest(path) -> List[str]:
    """Resolved camera paths of a local dataset manifest; relative entries are taken against the manifest's
    folder; a remote entry is an error."""
    path = _local(path, "dataset manifest")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"dataset manifest does not exist: {path}")
    out = []
    with open(path, encoding="utf-8") as fh:
        for ln, raw in enumerate(fh, start=1):
            entry = raw.strip()
            if not entry:
                continue
            if "://" in entry:
                raise ViewManifestError(f"{path}:{ln}: expected a local camera JSON path, got {entry!r}")
            entry = os.path.expanduser(entry)
            if not os.path.isabs(entry):
                entry = os.path.join(os.path.dirname(path), entry)
            out.append(os.path.realpath(entry))
    if not out:
        raise ViewManifestError(f"dataset manifest is empty: {path}")
    return out


def frame_id(frame: dict, index: int) -> str:
    for key in ("frame_id", "id", "image_id"):
        if frame.get(key) is not None:
            return str(frame[key])
    if frame.get("file_path") is not None:
        return str(frame["file_path"])
    return str(index)


def scene_id(payload, camera_path: str) -> str:
    """``scene_id`` / ``id`` / ``name`` of the camera file when it has one.  Otherwise the folder name for camera
    files with a generic name (``opencv_cameras*.json``, ``cameras.json``, ``transforms.json``...; one level
    further up when that folder is the renderer namespace ``kai``), else the file's stem."""
    if isinstance(payload, dict):
        for key in ("scene_id", "id", "name"):
            if payload.get(key) not in (None, ""):
                return str(payload[key])
    folder, name = os.path.split(str(camera_path))
    stem = os.path.splitext(name)[0]
    parent = os.path.basename(folder)
    if (stem.lower() in _GENERIC_STEMS or stem.lower().startswith("opencv_camera")) and parent:
        if parent.lower() == "kai":
            return os.path.basename(os.path.dirname(folder))
        return parent
    return stem


def select_views(n_frames: int, num_views: int, seed: int, sid: str) -> List[int]:
    if num_views <= 0:
        raise ViewManifestError(f"num_views must be positive, got {num_views}")
    if n_frames < num_views:
        raise ViewManifestError(f"scene {sid!r} has {n_frames} frames, but {num_views} ordered views are required")
    s = int.from_bytes(hashlib.sha256(f"{seed}\0{sid}".encode("utf-8")).digest()[:8], "big")
    return random.Random(s).sample(range(n_frames), num_views)     # sample order is kept: views are not sorted


def _read_camera(path: str):
    if not os.path.isfile(path):
        raise FileNotFoundError(f"camera JSON does not exist: {path}")
    with open(path, "rb") as fh:
        raw = fh.read()
    try:
        payload = json.loads(raw)
    except json.JSONDecodeError as exc:
        raise ViewManifestError(f"invalid camera JSON {path}: {exc}") from exc
    if not isinstance(payload, dict) or not isinstance(payload.get("frames"), list):
        raise ViewManifestError(f"camera JSON must be an object with a list-valued 'frames': {path}")
    return payload, hashlib.sha256(raw).hexdigest()


def _selection_digest(scenes) -> str:
    return hashlib.sha256(json.dumps(scenes, sort_keys=True).encode()).hexdigest()


def build_view_manifest(manifest, num_views: int = DEFAULT_NUM_VIEWS, seed: int = DEFAULT_VIEW_SEED,
                        dataset: str = "", unique: bool = False) -> Dict:
    """The frozen selection as a dictionary (not written).  Two entries that resolve to the same scene id are an
    error unless ``unique`` is given, which keeps the first of each camera path (manifests that list a scene several
    times to fill a training batch)."""
    manifest = _local(manifest, "dataset manifest")
    cameras = read_local_manifest(manifest)
    if unique:
        cameras = list(dict.fromkeys(cameras))
    with open(manifest, "rb") as fh:
        source_digest = hashlib.sha256(fh.read()).hexdigest()
    scenes, seen = [], {}
    for i, cam in enumerate(cameras):
        payload, digest = _read_camera(cam)
        sid = scene_id(payload, cam)
        if sid in seen:
            raise ViewManifestError(f"duplicate scene_id {sid!r}: {seen[sid]} and {cam}")
        seen[sid] = cam
        picks = select_views(len(payload["frames"]), num_views, seed, sid)
        scenes.append({"scene_index": i, "scene_id": sid, "camera_path": cam, "camera_sha256": digest,
                       "frame_indices": picks, "frame_ids": [frame_id(payload["frames"][j], j) for j in picks]})
    return {"schema_version": SCHEMA_VERSION, "dataset": str(dataset), "seed": int(seed), "num_views": int(num_views),
            "selection_method": SELECTION_METHOD, "source_manifest": manifest,
            "source_manifest_sha256": source_digest,
            "view_semantics": {"input": 0, "targets": list(range(1, num_views))},
            "scenes": scenes, "selection_sha256": _selection_digest(scenes)}


def _is_count(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def validate_view_manifest(doc, expected_num_views: Optional[int] = None) -> Dict:
    if not isinstance(doc, dict):
        raise ViewManifestError("view manifest must be a JSON object")
    if doc.get("schema_version") != SCHEMA_VERSION:
        raise ViewManifestError(f"unsupported view manifest schema_version {doc.get('schema_version')!r}; "
                                f"expected {SCHEMA_VERSION}")
    nv = doc.get("num_views")
    if not _is_count(nv) or nv <= 0:
        raise ViewManifestError(f"view manifest num_views must be a positive integer, got {nv!r}")
    if expected_num_views is not None and nv != expected_num_views:
        raise ViewManifestError(f"view manifest contains {nv} views; expected {expected_num_views}")
    sem = doc.get("view_semantics")
    if not isinstance(sem, dict) or sem.get("input") != 0:
        raise ViewManifestError("view manifest must designate View 0 as input")
    if sem.get("targets") != list(range(1, nv)):
        raise ViewManifestError(f"view manifest targets must be View 1..{nv - 1}")
    scenes = doc.get("scenes")
    if not isinstance(scenes, list) or not scenes:
        raise ViewManifestError("view manifest must contain at least one scene")
    seen = set()
    for i, entry in enumerate(scenes):
        where = f"scenes[{i}]"
        if not isinstance(entry, dict):
            raise ViewManifestError(f"{where} must be an object")
        if entry.get("scene_index") != i:
            raise ViewManifestError(f"{where}.scene_index must be {i}, got {entry.get('scene_index')!r}")
        sid = entry.get("scene_id")
        if not isinstance(sid, str) or not sid:
            raise ViewManifestError(f"{where}.scene_id must be a non-empty string")
        if sid in seen:
            raise ViewManifestError(f"duplicate scene_id {sid!r}")
        seen.add(sid)
        idx = entry.get("frame_indices")
        if not isinstance(idx, list) or len(idx) != nv or any(not _is_count(v) or v < 0 for v in idx):
            raise ViewManifestError(f"{where}.frame_indices must contain {nv} non-negative integers")
        if len(set(idx)) != nv:
            raise ViewManifestError(f"{where}.frame_indices must be unique")
        ids = entry.get("frame_ids")
        if not isinstance(ids, list) or len(ids) != nv or any(not isinstance(v, str) for v in ids):
            raise ViewManifestError(f"{where}.frame_ids must contain {nv} strings")
    if doc.get("selection_sha256") and doc["selection_sha256"] != _selection_digest(scenes):
        raise ViewManifestError("view manifest was edited after it was frozen (selection checksum mismatch)")
    return doc


def load_view_manifest(path, expected_num_views: Optional[int] = None) -> Dict:
    path = _local(path, "view manifest")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"view manifest does not exist: {path}")
    try:
        with open(path, encoding="utf-8") as fh:
            doc = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ViewManifestError(f"invalid view manifest JSON {path}: {exc}") from exc
    return validate_view_manifest(doc, expected_num_views)


def write_view_manifest(doc: Dict, output, overwrite: bool = False) -> str:
    validate_view_manifest(doc)
    output = _local(output, "view manifest output")
    if os.path.exists(output) and not overwrite:
        raise FileExistsError(f"refusing to overwrite existing view manifest: {output}; pass --force to replace it")
    os.makedirs(os.path.dirname(output) or ".", exist_ok=True)
    tmp = os.path.join(os.path.dirname(output), f".{os.path.basename(output)}.tmp")
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(doc, fh, indent=2, sort_keys=True)
        fh.write("\n")
    os.replace(tmp, output)
    return output


class FixedViewDataset(Dataset):
    """Scenes of a frozen view manifest, each returned with exactly its frozen, ordered views.

    With ``dataset_manifest`` the camera files are taken from it, entry by entry (a dataset that moved since the
    views were frozen); otherwise from the ``camera_path`` recorded in the view manifest.  Before a scene is read its
    camera file is checked against the frozen record: scene id, content digest (``verify_camera_sha256``), frame
    count, frame ids.  A read error is fatal for that sample: no other scene is substituted."""

    def __init__(self, view_manifest: str, image_size: int, shard_index: int = 0, num_shards: int = 1,
                 max_scenes: int = 0, dataset_manifest: Optional[str] = None, verify_camera_sha256: bool = True,
                 expected_num_views: Optional[int] = None, load_threads: int = 8):
        if load_threads <= 0:
            raise ValueError(f"load_threads must be positive, got {load_threads}")
        doc = load_view_manifest(view_manifest, expected_num_views)
        scenes: List[Dict] = [dict(s) for s in doc["scenes"]]
        if dataset_manifest is not None:
            cameras = read_local_manifest(dataset_manifest)
            if len(cameras) != len(scenes):
                raise ViewManifestError(f"dataset manifest has {len(cameras)} scenes, but frozen view manifest has "
                                        f"{len(scenes)} scenes")
            for s, cam in zip(scenes, cameras):
                s["camera_path"] = cam
        self.scenes = scenes[shard_index::num_shards]           # strided shard first, then the smoke-run cut
        if max_scenes:
            self.scenes = self.scenes[:max_scenes]
        self.num_views = doc["num_views"]
        self.dataset = str(doc.get("dataset", ""))
        self.verify_camera_sha256 = verify_camera_sha256
        self._loader = NVSDataset.__new__(NVSDataset)
        self._loader.image_size = image_size
        self._loader.LOAD_THREADS = load_threads

    def __len__(self):
        return len(self.scenes)

    def metadata(self, idx: int) -> Dict:
        e = self.scenes[idx]
        return {"scene_index": e["scene_index"], "scene_id": e["scene_id"], "camera_path": e["camera_path"],
                "frame_indices": list(e["frame_indices"]), "frame_ids": list(e["frame_ids"])}

    def _check(self, entry: Dict) -> None:
        cam, sid = entry["camera_path"], entry["scene_id"]
        payload, digest = _read_camera(cam)
        found = scene_id(payload, cam)
        if found != sid:
            raise ViewManifestError(f"scene index {entry['scene_index']}: frozen scene_id is {sid!r}, but local "
                                    f"camera JSON resolves to {found!r}")
        if self.verify_camera_sha256 and entry.get("camera_sha256") and digest != entry["camera_sha256"]:
            raise ViewManifestError(f"scene {sid!r}: camera JSON changed after view selection (expected sha256 "
                                    f"{entry['camera_sha256']}, got {digest})")
        frames = payload["frames"]
        if max(entry["frame_indices"]) >= len(frames):
            raise ViewManifestError(f"scene {sid!r}: frozen frame index {max(entry['frame_indices'])} is outside "
                                    f"local frame count {len(frames)}")
        if [frame_id(frames[j], j) for j in entry["frame_indices"]] != entry["frame_ids"]:
            raise ViewManifestError(f"scene {sid!r}: local frame IDs do not match the frozen view manifest")

    def __getitem__(self, idx: int):
        entry = self.scenes[idx]
        self._check(entry)
        imgs, intr, poses = self._loader.load_views(entry["camera_path"], entry["frame_indices"])
        return {"image": imgs, "fxfycxcy": intr, "c2w": poses, "scene_id": entry["scene_id"]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Freeze deterministic view selections for evaluation.")
    ap.add_argument("--dataset-manifest", "--manifest", dest="manifest", required=True,
                    help="Local newline-delimited camera JSON manifest.")
    ap.add_argument("--dataset", default="", help="Dataset label recorded in the output (gso, dl3dv, ...).")
    ap.add_argument("--output", required=True, help="Output JSON path.")
    ap.add_argument("--num-views", type=int, default=DEFAULT_NUM_VIEWS)
    ap.add_argument("--seed", type=int, default=DEFAULT_VIEW_SEED)
    ap.add_argument("--unique", action="store_true", help="Keep the first of repeated manifest entries.")
    ap.add_argument("--force", action="store_true", help="Replace an existing output manifest.")
    args = ap.parse_args(argv)
    doc = build_view_manifest(args.manifest, args.num_views, args.seed, dataset=args.dataset, unique=args.unique)
    out = write_view_manifest(doc, args.output, overwrite=args.force)
    print(f"Wrote {len(doc['scenes'])} scenes x {doc['num_views']} views to {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
