"""Scene data for view synthesis.

* :class:`SyntheticScenes`: images of smoothed Gaussian noise clipped to [0, 1]; cameras sampled uniformly on a
  sphere of radius 2 looking at the origin with a 50 degree field of view (benchmarks, tests).
* :func:`make_toy_dataset`: procedural scenes on a circular orbit written to disk in the loader's format
  (uttt_nvs/data/make_toy_dataset.py:26-128).
* :class:`NVSDataset`: manifest of per-scene camera JSON files; samples ``num_views`` frames, resize-cover +
  centre-crop with the intrinsics fixed up, RGBA composited on white, ``c2w = inv(w2c)``
  (uttt_nvs/data/loader.py:77-240).  Returns ``fxfycxcy [V,4], c2w [V,4,4], image [V,3,H,W], index [V,2]``.
* :class:`ResumableDistributedSampler`: epoch-deterministic permutation with a one-shot skip for mid-epoch
  resume (uttt_nvs/train/sampler.py:6-37).
"""
from __future__ import annotations

import json
import math
import os
import random
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch
import torch.nn.functional as F
from torch.utils.data import Dataset, DistributedSampler

from . import manifests


def look_at_c2w(eye: torch.Tensor, target: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Right-handed camera-to-world matrices (x right, y down, z forward / OpenCV) for eyes [n, 3]."""
    target = torch.zeros_like(eye) if target is None else target
    z = F.normalize(target - eye, dim=-1)
    up = torch.tensor([0.0, 0.0, 1.0], device=eye.device).expand_as(eye)
    x = F.normalize(torch.cross(z, up, dim=-1), dim=-1)
    bad = x.norm(dim=-1, keepdim=True) < 1e-6
    x = torch.where(bad, torch.tensor([1.0, 0.0, 0.0], device=eye.device).expand_as(x), x)
    y = torch.cross(z, x, dim=-1)
    c2w = torch.eye(4, device=eye.device).repeat(eye.shape[0], 1, 1)
    c2w[:, :3, 0], c2w[:, :3, 1], c2w[:, :3, 2], c2w[:, :3, 3] = x, y, z, eye
    return c2w


def sphere_cameras(n: int, radius: float, generator: torch.Generator) -> torch.Tensor:
    v = torch.randn(n, 3, generator=generator)
    return look_at_c2w(F.normalize(v, dim=-1) * radius)


def smoothed_noise_images(n: int, size: int, generator: torch.Generator, sigma: float = 4.0) -> torch.Tensor:
    x = torch.randn(n, 3, size, size, generator=generator)
    k = int(4 * sigma) | 1
    ax = torch.arange(k) - k // 2
    g = torch.exp(-(ax.float() ** 2) / (2 * sigma ** 2))
    g = (g / g.sum()).view(1, 1, 1, k)
    x = x.reshape(n * 3, 1, size, size)
    x = F.conv2d(F.pad(x, (k // 2, k // 2, 0, 0), mode="reflect"), g)
    x = F.conv2d(F.pad(x, (0, 0, k // 2, k // 2), mode="reflect"), g.transpose(2, 3))
    x = x.view(n, 3, size, size)
    x = x / x.std().clamp_min(1e-6) * 0.25 + 0.5
    return x.clamp(0, 1)


class SyntheticScenes:
    """Infinite stream of scene batches in (pinned) host memory."""

    def __init__(self, batch_size: int, num_views: int, image_size: int, seed: int = 0, rank: int = 0,
                 fov_deg: float = 50.0, radius: float = 2.0, pin: bool = True):
        self.batch_size, self.num_views, self.image_size = batch_size, num_views, image_size
        self.seed, self.rank, self.step = seed, rank, 0
        self.fov, self.radius = fov_deg, radius
        self.pin = pin and torch.cuda.is_available()

    def __iter__(self):
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(hash((self.seed, self.rank, self.step)) % (2 ** 31))
        self.step += 1
        b, v, s = self.batch_size, self.num_views, self.image_size
        image = smoothed_noise_images(b * v, s, g).view(b, v, 3, s, s)
        c2w = sphere_cameras(b * v, self.radius, g).view(b, v, 4, 4)
        f = 0.5 * s / math.tan(math.radians(self.fov) / 2)
        fxfycxcy = torch.tensor([f, f, s / 2, s / 2]).expand(b, v, 4).contiguous()
        batch = {"image": image, "fxfycxcy": fxfycxcy, "c2w": c2w}
        return {k: (t.pin_memory() if self.pin else t) for k, t in batch.items()}

    def state_dict(self):
        return {"step": self.step}

    def load_state_dict(self, sd):
        self.step = int(sd["step"])


def make_toy_dataset(out_dir: str, num_scenes: int = 4, num_frames: int = 16, image_size: int = 64,
                     seed: int = 0, repeat: int = 1) -> str:
    """Procedural scenes (coloured discs on a gradient) seen from a circular orbit, in the loader's on-disk layout:
    ``scene_NNN/images/NNN.png``, one ``scene_NNN/opencv_cameras.json`` with per-frame ``fx fy cx cy w2c
    file_path`` (image paths relative to the camera file), and ``manifest.txt`` listing the absolute camera paths
    ``repeat`` times each (a manifest line is a sample, so a few scenes can fill a large global batch).
    Returns the manifest path."""
    from PIL import Image
    for name, flag, value in (("num_scenes", "scenes", num_scenes), ("num_frames", "views", num_frames),
                              ("image_size", "size", image_size), ("repeat", "repeat", repeat)):
        if type(value) is not int or value < 1:
            raise ValueError(f"{name} (--{flag}) must be a positive integer")
    out_dir = os.path.abspath(os.path.expanduser(out_dir))
    rng = np.random.default_rng(seed)
    manifest = []
    f = 0.5 * image_size / math.tan(math.radians(50) / 2)
    for s in range(num_scenes):
        scene_dir = os.path.join(out_dir, f"scene_{s:03d}")
        os.makedirs(os.path.join(scene_dir, "images"), exist_ok=True)
        centres = rng.uniform(-0.5, 0.5, size=(5, 3))
        colours = rng.uniform(0.2, 1.0, size=(5, 3))
        frames = []
        for i in range(num_frames):
            ang = 2 * math.pi * i / num_frames
            eye = torch.tensor([[2 * math.cos(ang), 2 * math.sin(ang), 0.6]])
            c2w = look_at_c2w(eye)[0]
            w2c = torch.linalg.inv(c2w)
            img = np.ones((image_size, image_size, 3), np.float32) * np.linspace(0.2, 0.8, image_size)[:, None, None]
            pts = (w2c[:3, :3].numpy() @ centres.T + w2c[:3, 3:].numpy()).T
            for p, col in sorted(zip(pts, colours), key=lambda pc: -pc[0][2]):
                if p[2] <= 0.1:
                    continue
                u, v = f * p[0] / p[2] + image_size / 2, f * p[1] / p[2] + image_size / 2
                r = 0.18 * f / p[2]
                yy, xx = np.mgrid[0:image_size, 0:image_size]
                img[(xx - u) ** 2 + (yy - v) ** 2 < r * r] = col
            rel = f"images/{i:03d}.png"
            Image.fromarray((img * 255).astype(np.uint8)).save(os.path.join(scene_dir, rel))
            frames.append({"fx": f, "fy": f, "cx": image_size / 2, "cy": image_size / 2, "w2c": w2c.tolist(),
                           "file_path": rel})
        jpath = os.path.join(scene_dir, "opencv_cameras.json")
        with open(jpath, "w", encoding="utf-8") as fh:
            json.dump({"scene_name": f"scene_{s:03d}", "frames": frames}, fh)
        manifest.append(jpath)
    mpath = os.path.join(out_dir, "manifest.txt")
    with open(mpath, "w", encoding="utf-8") as fh:
        fh.write("\n".join(manifest * repeat) + "\n")
    return mpath


class NVSDataset(Dataset):
    """One sample per manifest line: ``num_views`` frames of that scene drawn without replacement.

    ``max_num_objects`` keeps the first n scenes and repeats them so that the epoch length stays (about) what it
    was (uttt_nvs/data/loader.py:150-154).  A sample that cannot be read is replaced by another one; after
    ``MAX_CONSECUTIVE_FAILURES`` failures in a row the error is raised with the last failing path."""
    MAX_CONSECUTIVE_FAILURES = 100
    LOAD_THREADS = 8

    def __init__(self, manifest: str, num_views: int, image_size: int, max_num_objects: Optional[int] = None,
                 seed: int = 0):
        self.scenes = manifests.read_manifest(manifest)
        manifests.drop_clients()            # a client made here must not travel to worker processes
        if max_num_objects and int(max_num_objects) > 0 and self.scenes:
            total = len(self.scenes)
            kept = self.scenes[:int(max_num_objects)]
            self.scenes = kept * max(total // len(kept), 1)
        if not self.scenes:
            raise ValueError(f"empty manifest {manifest}")
        self.num_views, self.image_size, self.seed = num_views, image_size, seed

    def __len__(self):
        return len(self.scenes)

    def _load_frame(self, frame, base_dir: str = ""):
        from PIL import Image
        with manifests.open_file(manifests.frame_image(frame, base_dir)) as fh:
            img = Image.open(fh)
            img.load()
        if img.mode == "RGBA":
            bg = Image.new("RGBA", img.size, (255, 255, 255, 255))
            img = Image.alpha_composite(bg, img)
        img = img.convert("RGB")
        fx, fy, cx, cy = manifests.frame_intrinsics(frame)
        w, h = img.size
        s = self.image_size
        scale = max(s / w, s / h)                       # resize so the image covers the square, then centre-crop
        nw, nh = round(w * scale), round(h * scale)
        img = img.resize((nw, nh), Image.LANCZOS)
        left, top = (nw - s) // 2, (nh - s) // 2
        img = img.crop((left, top, left + s, top + s))
        fx, fy, cx, cy = fx * nw / w, fy * nh / h, cx * nw / w - left, cy * nh / h - top
        arr = torch.from_numpy(np.asarray(img, dtype=np.float32) / 255.0).permute(2, 0, 1)
        c2w = torch.linalg.inv(torch.tensor(frame["w2c"], dtype=torch.float32))
        return arr, torch.tensor([fx, fy, cx, cy], dtype=torch.float32), c2w

    def load_views(self, camera_path: str, picks):
        """The given frames of one scene, read by a small thread pool: (images, intrinsics, poses)."""
        frames = manifests.read_frames(camera_path)
        base = manifests.parent_of(camera_path)
        if len(picks) > 1 and self.LOAD_THREADS > 1:
            with ThreadPoolExecutor(max_workers=min(self.LOAD_THREADS, len(picks))) as pool:
                out = list(pool.map(lambda i: self._load_frame(frames[i], base), picks))
        else:
            out = [self._load_frame(frames[i], base) for i in picks]
        imgs, intr, poses = zip(*out)
        return torch.stack(imgs), torch.stack(intr), torch.stack(poses)

    def __getitem__(self, idx: int):
        failures = 0
        # a fresh draw of views every time a scene comes up: the stream depends on the dataset seed, the loader's
        # per-epoch worker seed and the number of samples this copy of the dataset has served
        self._served = getattr(self, "_served", 0) + 1
        rng = random.Random(hash((self.seed, torch.initial_seed(), idx, self._served)))
        while True:
            try:
                n_frames = len(manifests.read_frames(self.scenes[idx]))
                if n_frames < self.num_views:
                    raise ValueError("scene has too few frames")
                picks = rng.sample(range(n_frames), self.num_views)
                imgs, intr, poses = self.load_views(self.scenes[idx], picks)
                index = torch.tensor([[i, idx] for i in picks])           # (frame, scene): the scene id is last
                return {"image": imgs, "fxfycxcy": intr, "c2w": poses, "index": index}
            except Exception as exc:
                failures += 1
                if failures >= self.MAX_CONSECUTIVE_FAILURES:
                    raise RuntimeError(
                        f"Failed to load {failures} samples in a row; the last failing path was "
                        f"'{self.scenes[idx]}'. Check that the manifest is readable and that every path in it "
                        f"is reachable.") from exc
                idx = rng.randrange(len(self.scenes))


def check_manifest(manifest: str, min_views: int = 1, check_images: bool = False) -> List[str]:
    """Error lines of :func:`uttt_b200.nvs.manifests.validate_manifest` (empty when the manifest is sound)."""
    return manifests.validate_manifest(manifest, min_views, check_images)["errors"]


class ResumableDistributedSampler(DistributedSampler):
    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._skip = 0

    def set_resume_offset(self, num_samples: int) -> None:
        if num_samples < 0:
            raise ValueError("num_samples must be non-negative")
        self._skip = int(num_samples)

    def __iter__(self):
        indices = list(super().__iter__())
        skip, self._skip = self._skip, 0
        if skip:
            if skip >= len(indices):
                raise ValueError(f"Resume offset {skip} is not smaller than this rank's epoch length {len(indices)}")
            indices = indices[skip:]
        return iter(indices)

    def __len__(self) -> int:
        return max(self.num_samples - self._skip, 0)


def main(argv=None):
    """``python -m uttt_b200.nvs.data make-toy --output DIR [--num-scenes 16] [--num-frames 24] [--image-size 256]
    [--repeat 16] [--seed 9595]`` (the defaults of uttt_nvs/data/make_toy_dataset.py:99-110: 24 frames per scene are
    what the fixed-view evaluation needs); ``check-manifest MANIFEST [--min-views N] [--check-images]``; ``build-manifest --root DIR
    --output manifest.txt [--pattern "opencv_cameras*.json"] [--limit N]`` (the last two are also
    ``python -m uttt_b200.nvs.manifests check | build``)."""
    import argparse
    import sys
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("make-toy")
    a.add_argument("--output", "--out", dest="output", required=True)
    a.add_argument("--num-scenes", "--scenes", dest="num_scenes", type=int, default=16)
    a.add_argument("--num-frames", "--views", dest="num_frames", type=int, default=24)
    a.add_argument("--image-size", "--size", dest="image_size", type=int, default=256)
    a.add_argument("--repeat", type=int, default=16)
    a.add_argument("--seed", type=int, default=9595)
    b = sub.add_parser("check-manifest")
    b.add_argument("manifest")
    b.add_argument("--min-views", type=int, default=1)
    b.add_argument("--check-images", action="store_true")
    c = sub.add_parser("build-manifest")
    c.add_argument("--root", required=True)
    c.add_argument("--output", "--out", dest="output", required=True)
    c.add_argument("--pattern", default=manifests.CAMERA_PATTERN)
    c.add_argument("--limit", type=int, default=0)
    args = ap.parse_args(argv)
    if args.cmd == "make-toy":
        try:
            print(make_toy_dataset(args.output, args.num_scenes, args.num_frames, args.image_size, args.seed,
                                   args.repeat))
        except ValueError as exc:
            ap.error(str(exc))
    elif args.cmd == "check-manifest":
        sys.exit(manifests.main(["check", args.manifest, "--min-views", str(args.min_views)]
                                + (["--check-images"] if args.check_images else [])))
    else:
        sys.exit(manifests.main(["build", "--root", args.root, "--out", args.output, "--pattern", args.pattern,
                                 "--limit", str(args.limit)]))


if __name__ == "__main__":
    main()
