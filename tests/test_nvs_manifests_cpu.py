"""On-disk data contracts of the view-synthesis side: camera files, dataset manifests, preflight checker, manifest
builder / localizer, frozen view manifests.  The expectations are those of the reference's tests/test_nvs_cpu.py and
its docs/data-contracts.md; the files are written here by hand in the reference's layout."""
import hashlib
import json
import os
import random

import numpy as np
import pytest
import torch
from PIL import Image

from uttt_b200.nvs import manifests
from uttt_b200.nvs.data import NVSDataset, make_toy_dataset
from uttt_b200.nvs.eval import views
from uttt_b200.tools import check_manifest as check_tool


def _write_scene(root, name, n_frames=5, size=(40, 24), mode="RGB", camera_name="opencv_cameras.json", extra=None):
    """A scene in the reference's layout, written without this package's helpers."""
    folder = root / name
    (folder / "images").mkdir(parents=True)
    frames = []
    for i in range(n_frames):
        arr = np.full((size[1], size[0], len(mode)), 40 * i % 255, np.uint8)
        if mode == "RGBA":
            arr[..., 3] = 0                                          # fully transparent: composites to white
        Image.fromarray(arr, mode).save(folder / "images" / f"{i:03d}.png")
        w2c = np.eye(4)
        w2c[:3, 3] = [0.1 * i, 0.0, 2.5]
        frames.append({"fx": 30.0, "fy": 31.0, "cx": size[0] / 2, "cy": size[1] / 2, "w2c": w2c.tolist(),
                       "file_path": f"images/{i:03d}.png"})
    doc = {"frames": frames}
    doc.update(extra or {})
    cam = folder / camera_name
    cam.write_text(json.dumps(doc))
    return cam


def _manifest(root, cams, name="manifest.txt"):
    path = root / name
    path.write_text("\n".join(str(c) for c in cams) + "\n\n")
    return path


def test_loader_reads_the_reference_layout(tmp_path):
    cams = [_write_scene(tmp_path, f"s{i}", n_frames=6) for i in range(3)]
    ds = NVSDataset(str(_manifest(tmp_path, cams)), num_views=4, image_size=16)
    item = ds[1]
    assert item["image"].shape == (4, 3, 16, 16) and item["c2w"].shape == (4, 4, 4)
    assert item["index"].shape == (4, 2) and set(item["index"][:, 1].tolist()) == {1}      # scene id is last
    assert len(set(item["index"][:, 0].tolist())) == 4                                     # without replacement
    # 40x24 -> cover 16x16: scale 2/3 -> 27x16, crop 5 columns on the left
    fx, fy, cx, cy = item["fxfycxcy"][0].tolist()
    assert fx == pytest.approx(30 * 27 / 40) and fy == pytest.approx(31 * 16 / 24)
    assert cx == pytest.approx(20 * 27 / 40 - 5) and cy == pytest.approx(12 * 16 / 24)
    frame = item["index"][0, 0].item()
    torch.testing.assert_close(item["c2w"][0, :3, 3], torch.tensor([-0.1 * frame, 0.0, -2.5]))


def test_loader_composites_rgba_on_white_and_reads_older_frames(tmp_path):
    cam = _write_scene(tmp_path, "alpha", n_frames=2, mode="RGBA", size=(16, 16))
    ds = NVSDataset(str(_manifest(tmp_path, [cam])), num_views=2, image_size=16)
    assert ds[0]["image"].min() == 1.0
    doc = json.loads(cam.read_text())
    for fr in doc["frames"]:                                        # one list + absolute path: still accepted
        fr["fxfycxcy"] = [fr.pop("fx"), fr.pop("fy"), fr.pop("cx"), fr.pop("cy")]
        fr["image_path"] = str(cam.parent / fr.pop("file_path"))
    cam.write_text(json.dumps(doc))
    assert ds[0]["fxfycxcy"][0].tolist() == pytest.approx([30.0, 31.0, 8.0, 8.0])


def test_max_num_objects_keeps_the_epoch_length(tmp_path):
    cams = [_write_scene(tmp_path, f"s{i}", n_frames=2, size=(8, 8)) for i in range(7)]
    ds = NVSDataset(str(_manifest(tmp_path, cams)), 2, 8, max_num_objects=2)
    assert len(ds) == 6 and set(ds.scenes) == {str(cams[0]), str(cams[1])}
    assert len(NVSDataset(str(_manifest(tmp_path, cams)), 2, 8, max_num_objects=-1)) == 7


def test_unreadable_samples_are_replaced_then_reported(tmp_path):
    good = _write_scene(tmp_path, "good", n_frames=3, size=(8, 8))
    man = _manifest(tmp_path, [tmp_path / "gone.json", good, tmp_path / "gone2.json"])
    ds = NVSDataset(str(man), 2, 8)
    assert ds[0]["index"][0, 1].item() == 1                          # the readable scene was substituted
    bad = NVSDataset(str(_manifest(tmp_path, [tmp_path / "gone.json"], "bad.txt")), 2, 8)
    bad.MAX_CONSECUTIVE_FAILURES = 5
    with pytest.raises(RuntimeError, match="gone.json"):
        bad[0]


def test_toy_dataset_uses_the_reference_layout(tmp_path):
    man = make_toy_dataset(str(tmp_path / "toy"), num_scenes=2, num_frames=5, image_size=16, repeat=3)
    lines = manifests.read_manifest(man)
    assert len(lines) == 6 and len(set(lines)) == 2 and all(os.path.isabs(p) for p in lines)
    assert os.path.basename(lines[0]) == "opencv_cameras.json"
    frame = json.load(open(lines[0]))["frames"][0]
    assert {"fx", "fy", "cx", "cy", "w2c", "file_path"} <= set(frame) and not os.path.isabs(frame["file_path"])
    report = manifests.validate_manifest(man, min_views=5, check_images=True)
    assert report == {"entries": 6, "unique_scenes": 2, "duplicate_entries": 4, "images_checked": 10,
                      "decoded_images": True, "errors": []}
    with pytest.raises(ValueError):
        make_toy_dataset(str(tmp_path / "x"), num_scenes=0)
    for field, flag in (("num_scenes", "scenes"), ("num_frames", "views"), ("image_size", "size"), ("repeat", "repeat")):
        kw = dict(num_scenes=1, num_frames=2, image_size=8, repeat=1)
        kw[field] = 0
        with pytest.raises(ValueError, match=flag):
            make_toy_dataset(str(tmp_path / "absent"), **kw)
    assert not (tmp_path / "absent").exists()


def test_toy_cli_defaults_give_enough_views_for_the_fixed_view_evaluation(tmp_path, capsys):
    from uttt_b200.nvs import data as nvs_data
    nvs_data.main(["make-toy", "--out", str(tmp_path), "--scenes", "1", "--size", "8", "--repeat", "1"])
    man = capsys.readouterr().out.strip().splitlines()[-1]
    assert man == str(tmp_path / "manifest.txt")
    assert not manifests.validate_manifest(man, min_views=24)["errors"]
    with pytest.raises(SystemExit) as err:
        nvs_data.main(["build-manifest", "--root", str(tmp_path), "--out", str(tmp_path / "m2.txt"), "--limit", "-1"])
    assert err.value.code == 2 and not (tmp_path / "m2.txt").exists()
    w2c = np.asarray(json.load(open(tmp_path / "scene_000" / "opencv_cameras.json"))["frames"][0]["w2c"])
    rot = w2c[:3, :3]                                     # right-handed OpenCV camera that sees the origin in front
    np.testing.assert_allclose(rot @ rot.T, np.eye(3), atol=1e-5)
    assert np.linalg.det(rot) == pytest.approx(1.0, abs=1e-5) and w2c[2, 3] > 0


def test_checker_reports_each_kind_of_damage(tmp_path):
    cams = [_write_scene(tmp_path, f"s{i}", n_frames=4, size=(8, 8)) for i in range(6)]

    def damage(i, fn):
        doc = json.loads(cams[i].read_text())
        fn(doc["frames"])
        cams[i].write_text(json.dumps(doc))

    damage(0, lambda fr: fr[1].update(fx=-1.0))
    damage(1, lambda fr: fr[0].update(w2c=np.zeros((4, 4)).tolist()))
    damage(2, lambda fr: fr[2].update(file_path="images/nope.png"))
    damage(3, lambda fr: fr[0].update(w2c=np.eye(3).tolist()))
    (cams[4].parent / "images" / "001.png").write_bytes(b"not a png")
    man = _manifest(tmp_path, cams + ["s3://bucket/scene/opencv_cameras.json", str(tmp_path / "absent.json")])
    plain = manifests.validate_manifest(str(man), min_views=4)
    text = "\n".join(plain["errors"])
    assert len(plain["errors"]) == 6 and not plain["decoded_images"]
    for needle in ("positive fx/fy", "invertible homogeneous", "image not found", "finite and 4x4", "cloud objects",
                   "absent.json"):
        assert needle in text
    decoded = manifests.validate_manifest(str(man), min_views=4, check_images=True)
    assert len(decoded["errors"]) == 7                               # the corrupt image shows only when decoded
    assert len(manifests.validate_manifest(str(man), min_views=5)["errors"]) == 8
    with pytest.raises(ValueError):
        manifests.validate_manifest(str(man), min_views=0)
    empty = tmp_path / "empty.txt"
    empty.write_text("\n\n")
    with pytest.raises(ValueError, match="empty"):
        manifests.validate_manifest(str(empty))


def test_checker_command_line(tmp_path, capsys):
    cam = _write_scene(tmp_path, "s", n_frames=3, size=(8, 8))
    man = _manifest(tmp_path, [cam])
    assert check_tool.main([str(man), "--min-views", "3", "--check-images"]) == 0
    assert json.loads(capsys.readouterr().out)["images_checked"] == 3
    assert check_tool.main([str(man)]) == 1                          # default asks for 24 views
    with pytest.raises(SystemExit) as exc:
        check_tool.main([str(tmp_path / "no_such_manifest.txt")])
    assert exc.value.code == 2


def test_build_and_localize(tmp_path):
    data = tmp_path / "data"
    cams = [_write_scene(data, f"scene_{i}") for i in range(3)]
    _write_scene(data, "other", camera_name="transforms.json")
    found = manifests.scan_cameras(str(data))
    assert found == sorted(str(c) for c in cams)
    assert manifests.scan_cameras(str(data), limit=2) == found[:2]
    assert len(manifests.scan_cameras(str(data), pattern="*.json")) == 4
    with pytest.raises(FileNotFoundError):
        manifests.scan_cameras(str(tmp_path / "nowhere"))
    assert manifests.main(["build", "--root", str(data), "--out", str(tmp_path / "m" / "train.txt")]) == 0
    assert manifests.read_manifest(str(tmp_path / "m" / "train.txt")) == found
    assert manifests.main(["build", "--root", str(data), "--out", str(tmp_path / "n.txt"), "--pattern", "x*"]) == 1

    remote = tmp_path / "remote.txt"
    remote.write_text("".join(f"s3://bucket/prefix/scene_{i}/opencv_cameras.json\n" for i in range(3)))
    local = manifests.translate_manifest(str(remote), source_prefix="s3://bucket/prefix", local_root=str(data))
    assert local == [os.path.realpath(c) for c in cams]
    out = manifests.write_manifest(local, str(tmp_path / "local.txt"))
    with pytest.raises(FileExistsError):
        manifests.write_manifest(local, out)
    manifests.write_manifest(local[:1], out, overwrite=True)
    assert manifests.read_manifest(out) == local[:1]
    with pytest.raises(ValueError, match="does not start with"):
        manifests.translate_manifest(str(remote), source_prefix="gs://elsewhere", local_root=str(data))
    escape = tmp_path / "escape.txt"
    escape.write_text("s3://bucket/prefix/../../etc/passwd\n")
    with pytest.raises(ValueError, match="escapes"):
        manifests.translate_manifest(str(escape), source_prefix="s3://bucket/prefix", local_root=str(data),
                                     verify_exists=False)
    missing = tmp_path / "missing.txt"
    missing.write_text("s3://bucket/prefix/scene_9/opencv_cameras.json\n")
    with pytest.raises(FileNotFoundError):
        manifests.translate_manifest(str(missing), source_prefix="s3://bucket/prefix", local_root=str(data))
    twice = tmp_path / "twice.txt"
    twice.write_text(remote.read_text() * 2)
    with pytest.raises(ValueError, match="duplicate"):
        manifests.translate_manifest(str(twice), source_prefix="s3://bucket/prefix", local_root=str(data))


def test_remote_entries_name_the_missing_package(tmp_path):
    try:
        import boto3  # noqa: F401
        pytest.skip("boto3 is installed")
    except ImportError:
        pass
    with pytest.raises(RuntimeError, match="boto3"):
        manifests.open_file("s3://bucket/key.json")
    assert manifests.join_path("s3://b/scene", "images/0.png") == "s3://b/scene/images/0.png"
    assert manifests.parent_of("gs://b/scene/opencv_cameras.json") == "gs://b/scene"


def test_scene_ids_follow_the_dataset_conventions():
    assert views.scene_id({"scene_id": "abc"}, "/d/x/opencv_cameras.json") == "abc"
    assert views.scene_id({"name": "n"}, "/d/x/cameras.json") == "n"
    assert views.scene_id({}, "/d/dl3dv/1K_0001/opencv_cameras.json") == "1K_0001"
    assert views.scene_id({}, "/d/gso/Shoe_A/kai/opencv_cameras.json") == "Shoe_A"
    assert views.scene_id({}, "/d/scenes/lego_truck.json") == "lego_truck"
    assert views.frame_id({"file_path": "images/3.png"}, 3) == "images/3.png"
    assert views.frame_id({"image_id": 17, "file_path": "a.png"}, 3) == "17"
    assert views.frame_id({}, 3) == "3"


def test_view_selection_rule_is_the_published_one():
    """Restated from the rule alone: sha256("<seed>\\0<scene id>"), first 8 bytes big-endian, random.sample."""
    for seed, sid, n, k in ((9595, "Shoe_A", 40, 24), (1, "scene_003", 30, 6)):
        s = int.from_bytes(hashlib.sha256(f"{seed}\0{sid}".encode()).digest()[:8], "big")
        assert views.select_views(n, k, seed, sid) == random.Random(s).sample(range(n), k)
    assert views.select_views(40, 24, 9595, "Shoe_A") != views.select_views(40, 24, 9595, "Shoe_B")
    with pytest.raises(views.ViewManifestError):
        views.select_views(10, 24, 9595, "x")


def test_frozen_views_round_trip_and_guard_against_drift(tmp_path):
    data = tmp_path / "data"
    cams = [_write_scene(data, f"scene_{i}", n_frames=8, size=(8, 8)) for i in range(3)]
    man = _manifest(tmp_path, cams)
    doc = views.build_view_manifest(str(man), num_views=4, seed=9595, dataset="toy")
    assert doc["schema_version"] == 1 and doc["selection_method"] == "per_scene_seeded_sample"
    assert doc["view_semantics"] == {"input": 0, "targets": [1, 2, 3]}
    assert doc["source_manifest_sha256"] == hashlib.sha256(man.read_bytes()).hexdigest()
    first = doc["scenes"][0]
    assert first["scene_id"] == "scene_0" and first["camera_sha256"] == hashlib.sha256(cams[0].read_bytes()).hexdigest()
    assert first["frame_ids"] == [f"images/{j:03d}.png" for j in first["frame_indices"]]
    # the order of the dataset manifest does not change a scene's views
    rev = views.build_view_manifest(str(_manifest(tmp_path, cams[::-1], "rev.txt")), num_views=4, seed=9595)
    assert {s["scene_id"]: s["frame_indices"] for s in rev["scenes"]} == \
           {s["scene_id"]: s["frame_indices"] for s in doc["scenes"]}

    out = views.write_view_manifest(doc, str(tmp_path / "views.json"))
    with pytest.raises(FileExistsError):
        views.write_view_manifest(doc, out)
    assert views.load_view_manifest(out, expected_num_views=4)["scenes"] == doc["scenes"]
    with pytest.raises(views.ViewManifestError, match="expected 24"):
        views.load_view_manifest(out, expected_num_views=24)

    # a manifest as the reference writes it (no selection digest) loads as well
    plain = {k: v for k, v in doc.items() if k != "selection_sha256"}
    (tmp_path / "plain.json").write_text(json.dumps(plain))
    ds = views.FixedViewDataset(str(tmp_path / "plain.json"), 8, dataset_manifest=str(man))
    assert len(ds) == 3 and ds[2]["image"].shape == (4, 3, 8, 8) and ds[2]["scene_id"] == "scene_2"
    assert ds.metadata(1)["frame_indices"] == doc["scenes"][1]["frame_indices"]

    for breakage, needle in (
            (lambda d: d.update(schema_version=2), "schema_version"),
            (lambda d: d["view_semantics"].update(input=1), "View 0"),
            (lambda d: d["scenes"][1].update(scene_index=5), "scene_index"),
            (lambda d: d["scenes"][1].update(scene_id="scene_0"), "duplicate"),
            (lambda d: d["scenes"][0]["frame_indices"].__setitem__(0, d["scenes"][0]["frame_indices"][1]), "unique"),
            (lambda d: d["scenes"][0].update(frame_ids=[1, 2, 3, 4]), "strings"),
            (lambda d: d.update(scenes=[]), "at least one scene")):
        broken = json.loads(json.dumps(plain))
        breakage(broken)
        with pytest.raises(views.ViewManifestError, match=needle):
            views.validate_view_manifest(broken)
    edited = json.loads(json.dumps(doc))
    edited["scenes"][0]["frame_indices"] = edited["scenes"][0]["frame_indices"][::-1]
    with pytest.raises(views.ViewManifestError, match="edited"):
        views.validate_view_manifest(edited)

    # drift of the data under a frozen selection is fatal for the sample
    with pytest.raises(views.ViewManifestError, match="scenes"):
        views.FixedViewDataset(out, 8, dataset_manifest=str(_manifest(tmp_path, cams[:2], "short.txt")))
    swapped = views.FixedViewDataset(out, 8, dataset_manifest=str(_manifest(tmp_path, cams[::-1], "swap.txt")))
    with pytest.raises(views.ViewManifestError, match="resolves to"):
        swapped[0]
    cams[1].write_text(cams[1].read_text() + " ")
    ds = views.FixedViewDataset(out, 8)
    with pytest.raises(views.ViewManifestError, match="changed after view selection"):
        ds[1]
    assert views.FixedViewDataset(out, 8, verify_camera_sha256=False)[1]["image"].shape[0] == 4
    payload = json.loads(cams[2].read_text())
    payload["frames"] = payload["frames"][::-1]
    cams[2].write_text(json.dumps(payload))
    with pytest.raises(views.ViewManifestError, match="frame IDs"):
        views.FixedViewDataset(out, 8, verify_camera_sha256=False)[2]
    os.remove(data / "scene_0" / "images" / f"{doc['scenes'][0]['frame_indices'][0]:03d}.png")
    with pytest.raises(OSError):
        ds[0]                                                        # no other scene is substituted

    dup = _manifest(tmp_path, [cams[0], cams[0]], "dup.txt")
    with pytest.raises(views.ViewManifestError, match="duplicate"):
        views.build_view_manifest(str(dup), num_views=4)
    assert len(views.build_view_manifest(str(dup), num_views=4, unique=True)["scenes"]) == 1
    with pytest.raises(views.ViewManifestError, match="local"):
        views.build_view_manifest("s3://bucket/manifest.txt")


def test_views_are_redrawn_every_time_a_scene_comes_up(tmp_path):
    cam = _write_scene(tmp_path, "s", n_frames=12, size=(8, 8))
    ds = NVSDataset(str(_manifest(tmp_path, [cam])), num_views=4, image_size=8)
    draws = {tuple(ds[0]["index"][:, 0].tolist()) for _ in range(6)}
    assert len(draws) > 1
    loader = torch.utils.data.DataLoader(ds, batch_size=1, num_workers=2)
    epochs = [tuple(next(iter(loader))["index"][0, :, 0].tolist()) for _ in range(4)]
    assert len(set(epochs)) > 1                               # worker copies start afresh each epoch, their seeds do not
