"""MVBench path of the quality tools on synthetic task files and ZIP archives: population and record
contract, repeated-media groups, member-wise extraction (local archive and HTTP range reads), exclusions,
verification."""

import hashlib
import http.server
import io
import json
import threading
import zipfile

import pytest

from prism_infer_b200.analysis import mvbench
from prism_infer_b200.analysis.identity import canonical_json_sha256
from prism_infer_b200.utils import build_mvbench_repeated_subset as subset_tool
from prism_infer_b200.utils import materialize_mvbench_media as media_tool


def _zip_bytes(members: dict[str, bytes]) -> bytes:
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w", zipfile.ZIP_DEFLATED) as z:
        for name, data in members.items():
            z.writestr(name, data)
    return buf.getvalue()


CLIPS = {"clips/a.mp4": b"A" * 3000, "clips/b.mp4": b"B" * 4100, "clips/c.mp4": b"C" * 10,
         "shots/s1/00001.jpg": b"f1" * 300, "shots/s1/00002.jpg": b"f2" * 300, "shots/s2/00001.jpg": b"g1" * 100}


@pytest.fixture()
def dataset(tmp_path):
    star = _zip_bytes({k: v for k, v in CLIPS.items() if k.startswith("clips/")})
    tv = _zip_bytes({k: v for k, v in CLIPS.items() if k.startswith("shots/")})
    archives = tmp_path / "video"
    archives.mkdir()
    (archives / "star.zip").write_bytes(star)
    (archives / "tv.zip").write_bytes(tv)
    media_map = {
        "schema_version": 1, "dataset_revision": "rev-1",
        "archives": {"star.zip": {"repository_path": "video/star.zip", "bytes": len(star), "sha256": hashlib.sha256(star).hexdigest()},
                     "tv.zip": {"repository_path": "video/tv.zip", "bytes": len(tv), "sha256": hashlib.sha256(tv).hexdigest()}},
        "tasks": {"action_sequence": {"archive": "star.zip", "media_prefix": "clips", "media_type": "video", "uses_temporal_bound": True},
                  "object_interaction": {"archive": "star.zip", "media_prefix": "clips", "media_type": "video", "uses_temporal_bound": True},
                  "episodic_reasoning": {"archive": "tv.zip", "media_prefix": "shots", "media_type": "frames", "uses_temporal_bound": False},
                  "fine_grained_pose": {"archive": None, "media_prefix": "ntu", "media_type": "video", "uses_temporal_bound": False,
                                        "availability": "manual_ntu_rgbd_license_required"}},
    }
    (tmp_path / "map.json").write_text(json.dumps(media_map))
    q = lambda video, n, **kw: {"video": video, "question": f"what happens {n}?", "candidates": ["x", "y", "z"], "answer": "y", **kw}
    tasks = {
        "action_sequence": [q("a.mp4", 0, start=0.0, end=4.0), q("a.mp4", 1, start=0.0, end=4.0), q("a.mp4", 2, start=4.0, end=9.5),
                            q("b.mp4", 3, start=1.0, end=2.0)],
        "object_interaction": [q("a.mp4", 0, start=0.0, end=4.0), q("gone.mp4", 1, start=0.0, end=1.0), q("gone.mp4", 2, start=0.0, end=1.0)],
        "episodic_reasoning": [q("s1", 0), q("s1", 1), q("s2", 2)],
        "fine_grained_pose": [q("p.avi", 0), q("p.avi", 1)],
    }
    jd = tmp_path / "json"
    jd.mkdir()
    for t, rows in tasks.items():
        (jd / f"{t}.json").write_text(json.dumps(rows))
    return tmp_path


def test_population_records_and_their_validation(dataset):
    mm = mvbench.MediaMap.load(dataset / "map.json")
    pop = mvbench.Population.load(dataset / "json", mm)
    assert len(pop.sample_ids) == 12 and pop.sample_ids[0] == "action_sequence|a.mp4|0"
    r = pop.records["action_sequence|a.mp4|2"]
    assert r["temporal_bound"] == {"start": 4.0, "end": 9.5} and r["answer_index"] == 1
    m = r["media"][0]
    assert m["archive_member_path"] == "clips/a.mp4" and m["materialization_status"] == mvbench.PENDING_ARCHIVE and m["sha256"] is None
    assert m["archive"]["name"] == "star.zip"
    manual = pop.records["fine_grained_pose|p.avi|0"]["media"][0]
    assert manual["materialization_status"] == mvbench.PENDING_MANUAL and "archive" not in manual
    assert pop.records["episodic_reasoning|s1|0"]["temporal_bound"] is None
    spec = mm.tasks["action_sequence"]
    for bad in ({"video": "a.mp4", "question": "q", "candidates": ["x"], "answer": "w", "start": 0, "end": 1},
                {"video": "a.mp4", "question": "q", "candidates": ["x"], "answer": "x", "start": 2, "end": 1},
                {"video": "a.mp4", "question": "q", "candidates": ["x"], "answer": "x", "start": True, "end": 3},
                {"video": "", "question": "q", "candidates": ["x"], "answer": "x", "start": 0, "end": 1},
                {"video": "a.mp4", "question": "q", "candidates": [], "answer": "x", "start": 0, "end": 1}):
        with pytest.raises(ValueError):
            mvbench.question_record(bad, index=0, media=spec, archives=mm.archives)
    with pytest.raises(ValueError):
        mvbench.sample_id("t|x", "v", 0)
    (dataset / "json" / "extra_task.json").write_text("[]")
    with pytest.raises(ValueError, match="extra=\\['extra_task'\\]"):
        mvbench.Population.load(dataset / "json", mm)


def test_repeated_media_groups_are_exact_and_ordered(dataset):
    mm = mvbench.MediaMap.load(dataset / "map.json")
    pop = mvbench.Population.load(dataset / "json", mm)
    records, groups = mvbench.repeated_media_groups([pop.records[s] for s in pop.sample_ids])
    by_ids = {tuple(g["sample_ids"]) for g in groups}
    # a.mp4 with window 0-4 is asked three times across two tasks; the 4-9.5 window and b.mp4 only once
    assert ("action_sequence|a.mp4|0", "action_sequence|a.mp4|1", "object_interaction|a.mp4|0") in by_ids
    assert ("object_interaction|gone.mp4|1", "object_interaction|gone.mp4|2") in by_ids
    assert ("episodic_reasoning|s1|0", "episodic_reasoning|s1|1") in by_ids
    assert ("fine_grained_pose|p.avi|0", "fine_grained_pose|p.avi|1") in by_ids
    assert len(groups) == 4 and len(records) == 9
    assert [g["source_contract_sha256"] for g in groups] == sorted(g["source_contract_sha256"] for g in groups)
    assert [r["sample_id"] for r in records] == [s for g in groups for s in g["sample_ids"]]
    for g in groups:
        assert g["source_contract_sha256"] == canonical_json_sha256(g["source_contract"])
    with pytest.raises(ValueError, match="no two"):
        mvbench.repeated_media_groups([pop.records["action_sequence|b.mp4|3"]])


def test_subset_build_then_local_extraction_exclusions_and_verify(dataset):
    out = dataset / "out"
    manifest = subset_tool.build(json_dir=dataset / "json", media_map_path=dataset / "map.json", out_root=out, revision="rev-1")
    assert manifest["repeated_media"]["groups"] == 4 and manifest["evaluation_subset"]["status"] == "pending"
    assert manifest["pending_media_plan"]["selected_samples_by_archive"] == {"star.zip": 5, "tv.zip": 2}
    assert manifest["pending_media_plan"]["manual_source_samples"] == 2
    with pytest.raises(FileExistsError):
        subset_tool.build(json_dir=dataset / "json", media_map_path=dataset / "map.json", out_root=out)
    with pytest.raises(ValueError, match="revision"):
        subset_tool.build(json_dir=dataset / "json", media_map_path=dataset / "map.json", out_root=dataset / "o2", revision="other")

    inv = media_tool.materialize(root=out, archive_dir=str(dataset / "video"), inventory_only=True)
    assert inv["archives"]["star.zip"]["unique_members"] == 1 and inv["archives"]["star.zip"]["missing_members"] == ["clips/gone.mp4"] * 2
    assert inv["archives"]["tv.zip"]["unique_members"] == 2
    assert not (out / "media").exists()

    first = media_tool.materialize(root=out, archive_dir=str(dataset / "video"), only=["star.zip"], check_archive_sha256=True)
    assert first["evaluation_subset"] == {"status": "pending", "eligible_samples": 3, "excluded_samples": 2, "pending_samples": 4}
    rep = media_tool.materialize(root=out, archive_dir=str(dataset / "video"), exclude_manual=True)
    assert rep["excluded_manual_sources"] == 2
    assert rep["evaluation_subset"] == {"status": "complete", "eligible_samples": 5, "excluded_samples": 4, "pending_samples": 0}
    final = json.loads((out / "mvbench_test.manifest.json").read_text())
    assert final["materialization_status"] == "complete_with_protocol_exclusions"
    assert final["pending_media_plan"] == {"selected_samples_by_archive": {}, "manual_source_samples": 0, "full_archive_download_bytes": 0}
    records = [json.loads(l) for l in (out / "mvbench_test.records.jsonl").read_text().splitlines()]
    video = next(r for r in records if r["sample_id"] == "action_sequence|a.mp4|0")["media"][0]
    digest = hashlib.sha256(CLIPS["clips/a.mp4"]).hexdigest()
    assert video["sha256"] == digest and video["identity_kind"] == "file_sha256"
    assert video["materialized_path"] == f"media/mvbench_test/{digest[:2]}/{digest}.mp4"
    assert (out / video["materialized_path"]).read_bytes() == CLIPS["clips/a.mp4"]
    frames = next(r for r in records if r["sample_id"] == "episodic_reasoning|s1|1")["media"][0]
    assert frames["identity_kind"] == "canonical_frame_manifest_sha256" and frames["materialized_path"] is None
    assert [f["archive_member_path"] for f in frames["frames"]] == ["shots/s1/00001.jpg", "shots/s1/00002.jpg"]
    assert frames["sha256"] == canonical_json_sha256([{"archive_member_path": f["archive_member_path"], "sha256": f["sha256"]} for f in frames["frames"]])
    gone = next(r for r in records if r["sample_id"] == "object_interaction|gone.mp4|1")["media"][0]
    assert gone["materialization_status"] == mvbench.EXCLUDED_MISSING and gone["sha256"] is None
    assert media_tool.verify(out) == {"records": 9, "unique_media_files": 3, "bytes": 3000 + 600 + 600}
    # a damaged file is caught, both by verify and by a repeated extraction
    path = out / video["materialized_path"]
    path.write_bytes(b"Z" * 3000)
    with pytest.raises(OSError, match="mismatch"):
        media_tool.verify(out)


def test_wrong_archive_size_or_suffix_is_refused(dataset):
    out = dataset / "out"
    subset_tool.build(json_dir=dataset / "json", media_map_path=dataset / "map.json", out_root=out)
    (dataset / "video" / "star.zip").write_bytes((dataset / "video" / "star.zip").read_bytes() + b"\0")
    with pytest.raises(ValueError, match="the media map records"):
        media_tool.materialize(root=out, archive_dir=str(dataset / "video"), only=["star.zip"])
    bad = _zip_bytes({"clips/a.mp4.exe": b"x"})
    with mvbench.ArchiveExtractor(io.BytesIO(bad), name="bad.zip", root=out) as ex:
        media = {"archive_member_path": "clips/a.mp4.exe", "media_type": "video"}
        with pytest.raises(ValueError, match="not a video file"):
            ex.materialize(media)


class _Ranges(http.server.BaseHTTPRequestHandler):
    files: dict[str, bytes] = {}
    served = 0

    def do_GET(self):  # noqa: N802
        data = self.files.get(self.path.split("?")[0])
        if data is None:
            self.send_error(404)
            return
        start, end = (int(x) for x in self.headers["Range"].split("=")[1].split("-"))
        end = min(end, len(data) - 1)
        body = data[start:end + 1]
        type(self).served += len(body)
        self.send_response(206)
        self.send_header("Content-Range", f"bytes {start}-{end}/{len(data)}")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def log_message(self, *a):
        pass


def test_extraction_over_http_range_reads(dataset):
    out = dataset / "out"
    subset_tool.build(json_dir=dataset / "json", media_map_path=dataset / "map.json", out_root=out)
    _Ranges.files = {f"/datasets/org/MVBench/resolve/rev-1/video/{n}": (dataset / "video" / n).read_bytes() for n in ("star.zip", "tv.zip")}
    _Ranges.served = 0
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _Ranges)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        rep = media_tool.materialize(root=out, endpoint=f"http://127.0.0.1:{srv.server_address[1]}", repository="org/MVBench",
                                     exclude_manual=True)
    finally:
        srv.shutdown()
    assert rep["evaluation_subset"]["eligible_samples"] == 5 and rep["archives"]["star.zip"]["range_requests"] >= 1
    assert media_tool.verify(out)["unique_media_files"] == 3
    with pytest.raises(ValueError, match="http"):
        media_tool.archive_url("ftp://x", "r", "v", "p")


def test_quality_runner_on_mvbench_frame_directories(tmp_path):
    """Subset -> extraction -> the working-set quality runner on the tiny model: questions over the same frame
    directory and time window form a group, the later ones hit the stored video prefix, answers are parsed the
    benchmark's way, excluded sources leave the run."""
    import importlib.util
    from pathlib import Path

    import numpy as np
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import working_set_quality as wsq
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    rng = np.random.default_rng(1)

    def png() -> bytes:
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, (32, 32, 3), dtype=np.uint8)).save(buf, format="PNG")
        return buf.getvalue()

    tv = _zip_bytes({f"shots/{d}/{i:05d}.png": png() for d in ("s1", "s2") for i in range(1, 9)})
    (tmp_path / "video").mkdir()
    (tmp_path / "video" / "tv.zip").write_bytes(tv)
    media_map = {"dataset_revision": "r", "archives": {"tv.zip": {"repository_path": "video/tv.zip", "bytes": len(tv), "sha256": hashlib.sha256(tv).hexdigest()}},
                 "tasks": {"episodic_reasoning": {"archive": "tv.zip", "media_prefix": "shots", "media_type": "frames", "uses_temporal_bound": True},
                           "fine_grained_pose": {"archive": None, "media_prefix": "ntu", "media_type": "video", "uses_temporal_bound": False}}}
    (tmp_path / "map.json").write_text(json.dumps(media_map))
    q = lambda video, n, **kw: {"video": video, "question": f"what happens {n}?", "candidates": ["x", "y", "z"], "answer": "z", **kw}
    (tmp_path / "json").mkdir()
    (tmp_path / "json" / "episodic_reasoning.json").write_text(json.dumps(
        [q("s1", 0, start=0.0, end=2.0), q("s1", 1, start=0.0, end=2.0), q("s2", 2, start=0.0, end=2.5), q("s2", 3, start=0.0, end=2.5),
         q("s2", 4, start=0.0, end=2.5)]))
    (tmp_path / "json" / "fine_grained_pose.json").write_text(json.dumps([q("p.avi", 0), q("p.avi", 1)]))
    out = tmp_path / "out"
    subset_tool.build(json_dir=tmp_path / "json", media_map_path=tmp_path / "map.json", out_root=out)
    media_tool.materialize(root=out, archive_dir=str(tmp_path / "video"), exclude_manual=True)

    spec = importlib.util.spec_from_file_location("bench_working_set_quality", Path(__file__).resolve().parents[1] / "benchmarks" / "bench_working_set_quality.py")
    runner = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runner)
    records = runner.load_records(out / "mvbench_test.records.jsonl")
    assert len(records) == 7 and all(runner.is_video_record(r) for r in records)
    records = runner.evaluable(records)
    assert len(records) == 5
    assert runner.verify_media(records, out)["unique_media_files"] == 16
    assert runner.prompt_for(records[0]).startswith("Question:what happens") and "(C) z" in runner.prompt_for(records[0])
    assert runner.score(records[0], "C. z")["correct"] and runner.score(records[0], "(C)")["parse_method"] == "embedded_label"
    assert not runner.score(records[0], "B")["correct"]
    plan = wsq.select_multi_question_groups(records, sampling_identity={"video_frames": 4, "frame_dir_fps": 3.0})
    assert sorted(it.group_size for it in plan) == [2, 2, 3, 3, 3]

    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)

    def make_engine(extra):
        return LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=128,
                   enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=True, **extra)

    run = tmp_path / "run"
    run.mkdir()
    rows = runner.run_stage("dense_prefix", plan, make_engine, out, run, max_tokens=3, resume=False, log=lambda _m: None, video_frames=4)
    assert [r["sample_id"] for r in rows] == [it.record["sample_id"] for it in plan]
    assert [r["prefix_hit"] for r in rows] == [it.question_index > 0 for it in plan]
    # eight frames at 3 fps, window 0 - 2 s -> frames 1..7 in four segments; the same indices for every question of the group
    by_group = {}
    for r in rows:
        by_group.setdefault(r["media_group_id"], set()).add((tuple(r["sampled_indices"]), r["sampled_rgb_identity_sha256"]))
    assert all(len(v) == 1 for v in by_group.values())
    assert all(len(r["sampled_indices"]) == 4 and r["parse_method"] in ("leading_label_period", "embedded_label", "unparseable") for r in rows)
    # the command-line entry end to end: both stages, summary with the identity of what went in
    final = tmp_path / "run_main"
    runner.main(["--records", str(out / "mvbench_test.records.jsonl"), "--media-root", str(out), "--out", str(final), "--model", "random:tiny",
                 "--device", "cpu", "--pages", "16", "--max-tokens", "2", "--video-frames", "4"])
    summary = json.loads((final / "summary.json").read_text())
    assert summary["samples"] == 5 and summary["groups"] == 2 and set(summary["stages"]) == {"dense_prefix", "compact_prefix"}
    assert summary["inputs"]["media_verified"]["unique_media_files"] == 16 and len(summary["inputs"]["records_file_sha256"]) == 64
    assert summary["provenance"]["source"] and summary["config"]["video_frames"] == 4
    assert summary["stages"]["dense_prefix"]["repeat_prefix_hits"] == summary["stages"]["dense_prefix"]["repeat_questions"] == 3


def test_video_file_record_is_sampled_inside_its_time_window(tmp_path):
    """A video-file source: extracted by content address, then decoded at the segment centres of the question's window."""
    cv2 = pytest.importorskip("cv2")
    import importlib.util
    from pathlib import Path

    import numpy as np

    clip = tmp_path / "clip.avi"
    w = cv2.VideoWriter(str(clip), cv2.VideoWriter_fourcc(*"MJPG"), 10.0, (32, 32))
    for i in range(40):
        w.write(np.full((32, 32, 3), 5 * i, np.uint8))
    w.release()
    star = _zip_bytes({"clips/a.avi": clip.read_bytes()})
    (tmp_path / "video").mkdir()
    (tmp_path / "video" / "star.zip").write_bytes(star)
    (tmp_path / "map.json").write_text(json.dumps({
        "dataset_revision": "r", "archives": {"star.zip": {"repository_path": "video/star.zip", "bytes": len(star), "sha256": hashlib.sha256(star).hexdigest()}},
        "tasks": {"action_sequence": {"archive": "star.zip", "media_prefix": "clips", "media_type": "video", "uses_temporal_bound": True}}}))
    (tmp_path / "json").mkdir()
    row = {"video": "a.avi", "question": "q?", "candidates": ["x", "y"], "answer": "x", "start": 1.0, "end": 3.0}
    (tmp_path / "json" / "action_sequence.json").write_text(json.dumps([row, dict(row, question="r?")]))
    out = tmp_path / "out"
    subset_tool.build(json_dir=tmp_path / "json", media_map_path=tmp_path / "map.json", out_root=out)
    media_tool.materialize(root=out, archive_dir=str(tmp_path / "video"))
    spec = importlib.util.spec_from_file_location("bench_working_set_quality", Path(__file__).resolve().parents[1] / "benchmarks" / "bench_working_set_quality.py")
    runner = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runner)
    records = runner.evaluable(runner.load_records(out / "mvbench_test.records.jsonl"))
    assert len(records) == 2 and runner.verify_media(records, out)["unique_media_files"] == 1
    frames, how = runner._load_frames(records[0], out, 4, 3.0)
    assert len(frames) == 4 and frames[0].shape == (32, 32, 3) and how["source_kind"] == "video_file"
    assert how["source_frame_count"] == 40 and all(10 <= i <= 30 for i in how["sampled_indices"])  # 1 s - 3 s at 10 fps
    assert how["sampled_indices"] == sorted(how["sampled_indices"])
    # brightness grows by 5 per frame: the decoded frames are the ones the indices name
    assert [int(round(float(f.mean()) / 5)) for f in frames] == how["sampled_indices"]
