"""Scene manifests on disk: reading, validating, building and relocating them.

The on-disk contract is the reference's (uttt_nvs/data/loader.py:170-200, docs/data-contracts.md): a manifest is a
UTF-8 text file with one camera-JSON path per non-empty line (local, ``s3://`` or ``gs://``); a camera JSON holds
``{"frames": [{"fx", "fy", "cx", "cy", "w2c", "file_path"}, ...]}`` where ``w2c`` is a 4x4 world-to-camera matrix
and ``file_path`` is resolved against the folder of the camera JSON.  Frames written by earlier versions of this
package (``fxfycxcy`` as one list, ``image_path`` absolute) are still read.

* :func:`open_file`: binary stream for a local path, an ``s3://`` object or a ``gs://`` blob (the cloud clients
  are created lazily in whichever process reads the entry, uttt_nvs/data/loader.py:25-75).
* :func:`validate_manifest`: the preflight check of tools/check_manifest.py:13-50, same report keys.
* :func:`scan_cameras`: manifest builder of uttt_nvs/data/build_manifest.py:49-112.
* :func:`translate_manifest` / :func:`write_manifest`: object-store manifest to verified local paths
  (uttt_nvs/eval/build_local_dataset_manifest.py:11-84).

    python -m uttt_b200.nvs.manifests check MANIFEST [--min-views 24] [--check-images]
    python -m uttt_b200.nvs.manifests build --root DIR|s3://..|gs://.. --out FILE [--pattern G] [--limit N]
    python -m uttt_b200.nvs.manifests localize --source-manifest F --source-prefix P --local-root D --output O
"""
from __future__ import annotations

import argparse
import fnmatch
import io
import json
import os
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

CAMERA_PATTERN = "opencv_cameras*.json"
_CLOUD = ("s3://", "gs://")
_clients: Dict[str, object] = {}


def is_remote(path: str) -> bool:
    return path.startswith(_CLOUD)


def _s3_client():
    if "s3" not in _clients:
        try:
            import boto3
            from botocore import UNSIGNED
            from botocore.config import Config
        except ImportError as exc:
            raise RuntimeError("reading s3:// entries needs the boto3 package") from exc
        _clients["s3"] = boto3.client("s3", config=Config(region_name=os.environ.get("AWS_REGION", "us-west-2"),
                                                          signature_version=UNSIGNED))
    return _clients["s3"]


def _gcs_client():
    if "gs" not in _clients:
        try:
            from google.cloud import storage
        except ImportError as exc:
            raise RuntimeError("reading gs:// entries needs the google-cloud-storage package") from exc
        _clients["gs"] = storage.Client()
    return _clients["gs"]


def drop_clients() -> None:
    """Forget the cloud clients (they do not survive being sent to data-loader worker processes)."""
    _clients.clear()


def open_file(path: str):
    """Binary, seekable stream of a local file, an ``s3://bucket/key`` object or a ``gs://bucket/blob``."""
    if path.startswith("s3://"):
        bucket, _, key = path[5:].partition("/")
        buf = io.BytesIO()
        _s3_client().download_fileobj(bucket, key, buf)
        buf.seek(0)
        return buf
    if path.startswith("gs://"):
        bucket, _, blob = path[5:].partition("/")
        return io.BytesIO(_gcs_client().bucket(bucket).blob(blob).download_as_bytes(timeout=60))
    return open(path, "rb")


def read_text(path: str) -> str:
    with open_file(path) as fh:
        data = fh.read()
    return data.decode("utf-8") if isinstance(data, bytes) else data


def read_manifest(path: str) -> List[str]:
    """Non-empty lines of a manifest, in order, duplicates kept (a line is one sample)."""
    return [ln.strip() for ln in read_text(path).splitlines() if ln.strip()]


def read_frames(camera_path: str) -> list:
    return json.loads(read_text(camera_path))["frames"]


def join_path(base: str, rel: str) -> str:
    if is_remote(rel) or os.path.isabs(rel):
        return rel
    if is_remote(base):
        return base.rstrip("/") + "/" + rel
    return os.path.join(base, rel)


def parent_of(camera_path: str) -> str:
    if is_remote(camera_path):
        return camera_path.rsplit("/", 1)[0]
    return os.path.dirname(camera_path)


def frame_intrinsics(frame: dict) -> Tuple[float, float, float, float]:
    if "fx" in frame:
        return float(frame["fx"]), float(frame["fy"]), float(frame["cx"]), float(frame["cy"])
    fx, fy, cx, cy = frame["fxfycxcy"]
    return float(fx), float(fy), float(cx), float(cy)


def frame_image(frame: dict, base_dir: str) -> str:
    if "file_path" in frame:
        return join_path(base_dir, frame["file_path"])
    return frame["image_path"]


def _check_frame(i: int, frame: dict, base_dir: str, check_images: bool) -> None:
    k = np.asarray(frame_intrinsics(frame), dtype=float)
    if not np.isfinite(k).all() or (k[:2] <= 0).any():
        raise ValueError(f"frame {i}: intrinsics must be finite with positive fx/fy")
    m = np.asarray(frame["w2c"], dtype=float)
    if m.shape != (4, 4) or not np.isfinite(m).all():
        raise ValueError(f"frame {i}: w2c must be finite and 4x4")
    if not np.allclose(m[3], [0, 0, 0, 1]) or abs(np.linalg.det(m)) < 1e-12:
        raise ValueError(f"frame {i}: w2c must be an invertible homogeneous transform")
    img = frame_image(frame, base_dir)
    if not os.path.isfile(img):
        raise ValueError(f"frame {i}: image not found: {img}")
    if check_images:
        from PIL import Image
        with Image.open(img) as im:
            im.verify()                     # structure of the file
        with Image.open(img) as im:
            im.load()                       # full decode (verify() leaves the object unusable)


def validate_manifest(path: str, min_views: int = 24, check_images: bool = False) -> dict:
    """Local preflight check.  Every distinct scene is checked once: at least ``min_views`` frames, finite
    intrinsics with positive focal lengths, a finite invertible homogeneous ``w2c``, the image file present (and
    decodable with ``check_images``).  Cloud entries are reported as errors, not skipped."""
    if min_views < 1:
        raise ValueError("min_views must be positive")
    entries = read_manifest(str(path))
    if not entries:
        raise ValueError("Manifest is empty")
    distinct = list(dict.fromkeys(entries))
    errors, images = [], 0
    for cam in distinct:
        try:
            if is_remote(cam):
                raise ValueError("local checker cannot validate cloud objects; stage this scene locally first")
            frames = read_frames(cam)
            if not isinstance(frames, list) or len(frames) < min_views:
                raise ValueError(f"frames must be a list with at least {min_views} views")
            base = parent_of(cam)
            for i, frame in enumerate(frames):
                _check_frame(i, frame, base, check_images)
                images += 1
        except (OSError, ValueError, KeyError, TypeError) as exc:
            errors.append(f"{cam}: {exc}")
    return {"entries": len(entries), "unique_scenes": len(distinct),
            "duplicate_entries": len(entries) - len(distinct), "images_checked": images,
            "decoded_images": bool(check_images), "errors": errors}


def scan_cameras(root: str, pattern: str = CAMERA_PATTERN, limit: int = 0) -> List[str]:
    """Sorted camera-JSON paths under a folder, an ``s3://`` prefix or a ``gs://`` prefix whose file name matches
    ``pattern``; local results are absolute so the manifest does not depend on the working directory."""
    if limit < 0:
        raise ValueError("limit must be non-negative")
    found: List[str] = []
    if root.startswith("s3://"):
        bucket, _, prefix = root[5:].partition("/")
        for page in _s3_client().get_paginator("list_objects_v2").paginate(Bucket=bucket, Prefix=prefix):
            for obj in page.get("Contents", []):
                if fnmatch.fnmatch(os.path.basename(obj["Key"]), pattern):
                    found.append(f"s3://{bucket}/{obj['Key']}")
    elif root.startswith("gs://"):
        bucket, _, prefix = root[5:].partition("/")
        for blob in _gcs_client().list_blobs(bucket, prefix=prefix):
            if fnmatch.fnmatch(os.path.basename(blob.name), pattern):
                found.append(f"gs://{bucket}/{blob.name}")
    else:
        top = os.path.abspath(os.path.expanduser(root))
        if not os.path.isdir(top):
            raise FileNotFoundError(f"Dataset root is not a directory: {top}")
        for folder, _dirs, names in os.walk(top):
            found.extend(os.path.join(folder, n) for n in names if fnmatch.fnmatch(n, pattern))
    found.sort()
    return found[:limit] if limit else found


def translate_manifest(source_manifest: str, *, source_prefix: str, local_root: str,
                       verify_exists: bool = True) -> List[str]:
    """Rewrites every entry ``<source_prefix>/<rel>`` to ``<local_root>/<rel>``.  Raises when an entry does not
    carry the prefix, would leave ``local_root`` (``..``), is missing on disk (``verify_exists``) or repeats."""
    src = os.path.realpath(os.path.expanduser(str(source_manifest)))
    root = os.path.realpath(os.path.expanduser(str(local_root)))
    if not os.path.isfile(src):
        raise FileNotFoundError(f"source manifest does not exist: {src}")
    if not source_prefix:
        raise ValueError("source_prefix must be non-empty")
    out: List[str] = []
    with open(src, encoding="utf-8") as fh:
        for ln, raw in enumerate(fh, start=1):
            entry = raw.strip()
            if not entry:
                continue
            if not entry.startswith(source_prefix):
                raise ValueError(f"{src}:{ln}: path does not start with {source_prefix!r}: {entry!r}")
            rel = entry[len(source_prefix):].lstrip("/")
            if not rel:
                raise ValueError(f"{src}:{ln}: source path has no relative suffix")
            local = os.path.realpath(os.path.join(root, rel))
            if os.path.commonpath([root, local]) != root:
                raise ValueError(f"{src}:{ln}: translated path escapes local root {root}: {local}")
            if verify_exists and not os.path.isfile(local):
                raise FileNotFoundError(f"{src}:{ln}: local camera JSON is missing: {local}")
            out.append(local)
    if not out:
        raise ValueError(f"source manifest has no non-empty entries: {src}")
    if len(set(out)) != len(out):
        raise ValueError("translated manifest contains duplicate camera paths")
    return out


def write_manifest(paths: Sequence[str], output: str, overwrite: bool = False) -> str:
    """Atomic write (temporary file + rename); refuses to replace an existing file unless ``overwrite``."""
    output = os.path.realpath(os.path.expanduser(str(output)))
    if os.path.exists(output) and not overwrite:
        raise FileExistsError(f"refusing to overwrite {output}; pass --force to replace it")
    os.makedirs(os.path.dirname(output) or ".", exist_ok=True)
    tmp = os.path.join(os.path.dirname(output), f".{os.path.basename(output)}.{os.getpid()}.tmp")
    with open(tmp, "w", encoding="utf-8") as fh:
        fh.writelines(f"{p}\n" for p in paths)
    os.replace(tmp, output)
    return output


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Scene manifests: check, build, localize.")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("check")
    c.add_argument("manifest")
    c.add_argument("--min-views", type=int, default=24)
    c.add_argument("--check-images", action="store_true")
    b = sub.add_parser("build")
    b.add_argument("--root", required=True)
    b.add_argument("--out", required=True)
    b.add_argument("--pattern", default=CAMERA_PATTERN)
    b.add_argument("--limit", type=int, default=0)
    t = sub.add_parser("localize")
    t.add_argument("--source-manifest", required=True)
    t.add_argument("--source-prefix", required=True)
    t.add_argument("--local-root", required=True)
    t.add_argument("--output", required=True)
    t.add_argument("--skip-existence-check", action="store_true")
    t.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    if args.cmd == "check":
        try:
            report = validate_manifest(args.manifest, args.min_views, args.check_images)
        except (OSError, ValueError) as exc:
            ap.error(str(exc))
        print(json.dumps(report, indent=2))
        return int(bool(report["errors"]))
    if args.cmd == "build":
        if args.limit < 0:
            ap.error("--limit must be non-negative")
        found = scan_cameras(args.root, args.pattern, args.limit)
        if not found:
            print(f"No files matching {args.pattern!r} under {args.root}.", file=sys.stderr)
            return 1
        write_manifest(found, args.out, overwrite=True)
        print(f"Wrote {len(found)} entries to {args.out}", file=sys.stderr)
        return 0
    paths = translate_manifest(args.source_manifest, source_prefix=args.source_prefix, local_root=args.local_root,
                               verify_exists=not args.skip_existence_check)
    out = write_manifest(paths, args.output, overwrite=args.force)
    print(f"Wrote {len(paths)} local camera paths to {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
