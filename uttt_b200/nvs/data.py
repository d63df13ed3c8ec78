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
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch
import torch.nn.functional as F
from torch.utils.data import Dataset, DistributedSampler


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
                     seed: int = 0) -> str:
    """Procedural scenes (coloured discs on a gradient) seen from a circular orbit; writes PNG frames, one camera
    JSON per scene and a manifest listing the JSON paths.  Returns the manifest path."""
    from PIL import Image
    rng = np.random.default_rng(seed)
    os.makedirs(out_dir, exist_ok=True)
    manifest = []
    f = 0.5 * image_size / math.tan(math.radians(50) / 2)
    for s in range(num_scenes):
        scene_dir = os.path.join(out_dir, f"scene_{s:04d}")
        os.makedirs(scene_dir, exist_ok=True)
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
            path = os.path.join(scene_dir, f"{i:03d}.png")
            Image.fromarray((img * 255).astype(np.uint8)).save(path)
            frames.append({"image_path": path, "fxfycxcy": [f, f, image_size / 2, image_size / 2],
                           "w2c": w2c.tolist()})
        jpath = os.path.join(scene_dir, "cameras.json")
        with open(jpath, "w") as fh:
            json.dump({"scene_name": f"scene_{s:04d}", "frames": frames}, fh)
        manifest.append(jpath)
    mpath = os.path.join(out_dir, "manifest.txt")
    with open(mpath, "w") as fh:
        fh.write("\n".join(manifest) + "\n")
    return mpath


class NVSDataset(Dataset):
    MAX_CONSECUTIVE_FAILURES = 100

    def __init__(self, manifest: str, num_views: int, image_size: int, max_num_objects: Optional[int] = None,
                 seed: int = 0):
        with open(manifest) as fh:
            self.scenes = [ln.strip() for ln in fh if ln.strip()]
        if max_num_objects:
            self.scenes = self.scenes[:max_num_objects]
        if not self.scenes:
            raise ValueError(f"empty manifest {manifest}")
        self.num_views, self.image_size, self.seed = num_views, image_size, seed

    def __len__(self):
        return len(self.scenes)

    def _load_frame(self, frame):
        from PIL import Image
        img = Image.open(frame["image_path"])
        if img.mode == "RGBA":
            bg = Image.new("RGBA", img.size, (255, 255, 255, 255))
            img = Image.alpha_composite(bg, img)
        img = img.convert("RGB")
        fx, fy, cx, cy = frame["fxfycxcy"]
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

    def __getitem__(self, idx: int):
        failures = 0
        rng = random.Random((self.seed, idx).__hash__())
        while True:
            try:
                with open(self.scenes[idx]) as fh:
                    scene = json.load(fh)
                frames = scene["frames"]
                if len(frames) < self.num_views:
                    raise ValueError("scene has too few frames")
                picks = rng.sample(range(len(frames)), self.num_views)
                imgs, intr, poses = zip(*[self._load_frame(frames[i]) for i in picks])
                index = torch.tensor([[idx, i] for i in picks])
                return {"image": torch.stack(imgs), "fxfycxcy": torch.stack(intr), "c2w": torch.stack(poses),
                        "index": index}
            except Exception:
                failures += 1
                if failures >= self.MAX_CONSECUTIVE_FAILURES:
                    raise
                idx = rng.randrange(len(self.scenes))


def check_manifest(manifest: str) -> List[str]:
    """Static validation of a manifest: every JSON parses, has frames with intrinsics, 4x4 poses and images."""
    problems = []
    with open(manifest) as fh:
        scenes = [ln.strip() for ln in fh if ln.strip()]
    for path in scenes:
        try:
            with open(path) as fh:
                scene = json.load(fh)
            for fr in scene["frames"]:
                if len(fr["fxfycxcy"]) != 4 or np.asarray(fr["w2c"]).shape != (4, 4):
                    problems.append(f"{path}: malformed camera")
                if not os.path.exists(fr["image_path"]):
                    problems.append(f"{path}: missing {fr['image_path']}")
        except Exception as exc:
            problems.append(f"{path}: {exc}")
    return problems


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
    """``python -m uttt_b200.nvs.data make-toy --output DIR [--num-scenes 4] [--num-frames 16] [--image-size 64]``
    ``python -m uttt_b200.nvs.data check-manifest MANIFEST``
    ``python -m uttt_b200.nvs.data build-manifest --root DIR --output manifest.txt [--pattern "**/cameras.json"]``"""
    import argparse
    import glob
    import sys
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("make-toy")
    a.add_argument("--output", required=True)
    a.add_argument("--num-scenes", type=int, default=4)
    a.add_argument("--num-frames", type=int, default=16)
    a.add_argument("--image-size", type=int, default=64)
    a.add_argument("--seed", type=int, default=0)
    b = sub.add_parser("check-manifest")
    b.add_argument("manifest")
    c = sub.add_parser("build-manifest")
    c.add_argument("--root", required=True)
    c.add_argument("--output", required=True)
    c.add_argument("--pattern", default="**/*.json")
    args = ap.parse_args(argv)
    if args.cmd == "make-toy":
        print(make_toy_dataset(args.output, args.num_scenes, args.num_frames, args.image_size, args.seed))
    elif args.cmd == "check-manifest":
        problems = check_manifest(args.manifest)
        for p in problems:
            print("ERROR", p)
        print(f"{len(problems)} problem(s)")
        sys.exit(1 if problems else 0)
    else:
        paths = sorted(os.path.abspath(p) for p in glob.glob(os.path.join(args.root, args.pattern), recursive=True))
        keep = []
        for p in paths:
            try:
                with open(p) as fh:
                    if "frames" in json.load(fh):
                        keep.append(p)
            except Exception:
                continue
        with open(args.output, "w") as fh:
            fh.write("\n".join(keep) + "\n")
        print(f"{len(keep)} scenes -> {args.output}")


if __name__ == "__main__":
    main()
