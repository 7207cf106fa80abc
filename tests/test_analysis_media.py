"""Video sampling, HTTP range reader, free-text scores, quality protocol validator (CPU)."""

import http.server
import io
import threading
import zipfile

import numpy as np
import pytest

from prism_infer_b200.analysis import http_range_reader as hrr
from prism_infer_b200.analysis import quality_protocol as qp
from prism_infer_b200.analysis import reference_quality as rq
from prism_infer_b200.analysis import video_sampling as vs


def test_segment_centre_indices_match_the_published_rule():
    # 100 frames, 8 samples: segment 12.375 -> centres 6, 18, 31, 43, 56, 68, 80, 93
    got = vs.uniform_segment_center_indices(first_index=0, max_index=99, frames=8, fps=25.0)
    seg = 99 / 8
    assert got == [int(seg / 2 + round(seg * i)) for i in range(8)] == [6, 18, 31, 43, 56, 68, 80, 93]
    bounded = vs.uniform_segment_center_indices(first_index=1, max_index=300, frames=4, fps=3.0, temporal_bound={"start": 10.0, "end": 20.0})
    assert bounded[0] >= 30 and bounded[-1] <= 60 and bounded == sorted(bounded)
    with pytest.raises(ValueError):
        vs.uniform_segment_center_indices(first_index=0, max_index=9, frames=2, fps=1.0, temporal_bound={"start": 50, "end": 60})
    with pytest.raises(ValueError):
        vs.uniform_segment_center_indices(first_index=0, max_index=9, frames=True, fps=1.0)


def test_frame_sequence_and_manifest_sampling(tmp_path):
    from PIL import Image

    rng = np.random.default_rng(0)
    frames = [rng.integers(0, 256, (8, 8, 3), dtype=np.uint8) for _ in range(20)]
    picked, rec = vs.sample_frame_sequence(frames, frames=4, fps=10.0)
    assert rec["sampled_indices"] == vs.uniform_segment_center_indices(first_index=0, max_index=19, frames=4, fps=10.0)
    assert all(np.array_equal(p, frames[i]) for p, i in zip(picked, rec["sampled_indices"]))
    records = []
    for i, f in enumerate(frames, 1):
        Image.fromarray(f).save(tmp_path / f"f{i}.png")
        records.append({"archive_member_path": f"clip/{i:05d}.jpg", "materialized_path": f"f{i}.png"})
    picked2, rec2 = vs.sample_frame_manifest(records, materialized_root=tmp_path, frames=4, fps=3.0)
    assert rec2["source_frame_count"] == 20 and all(1 <= i <= 20 for i in rec2["sampled_indices"])
    assert np.array_equal(picked2[0], frames[rec2["sampled_indices"][0] - 1])
    with pytest.raises(ValueError, match="gaps"):
        vs.sample_frame_manifest(records[:5] + records[6:], materialized_root=tmp_path, frames=2, fps=3.0)
    bad = [dict(records[0], materialized_path="../outside.png")]
    with pytest.raises(ValueError, match="escapes"):
        vs.sample_frame_manifest(bad, materialized_root=tmp_path, frames=1, fps=3.0)


class _RangeHandler(http.server.BaseHTTPRequestHandler):
    payload = b""
    hits = 0
    fail_first = 0

    def do_GET(self):  # noqa: N802
        cls = type(self)
        cls.hits += 1
        if cls.fail_first > 0:
            cls.fail_first -= 1
            self.send_response(503)
            self.end_headers()
            return
        rng = self.headers.get("Range")
        if rng is None or self.path == "/norange":
            self.send_response(200)
            self.send_header("Content-Length", str(len(cls.payload)))
            self.end_headers()
            self.wfile.write(cls.payload)
            return
        a, b = rng.split("=")[1].split("-")
        a, b = int(a), int(b)
        body = cls.payload[a:b + 1]
        self.send_response(206)
        self.send_header("Content-Range", f"bytes {a}-{b}/{len(cls.payload)}")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def log_message(self, *args):
        pass


@pytest.fixture()
def range_server():
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w", zipfile.ZIP_STORED) as z:
        for i in range(6):
            z.writestr(f"m{i}.bin", bytes([i]) * 5000)
    _RangeHandler.payload, _RangeHandler.hits, _RangeHandler.fail_first = buf.getvalue(), 0, 0
    srv = http.server.ThreadingHTTPServer(("127.0.0.1", 0), _RangeHandler)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield f"http://127.0.0.1:{srv.server_address[1]}"
    srv.shutdown()
    srv.server_close()


def test_http_range_reader_reads_one_zip_member_without_the_whole_archive(range_server):
    size = len(_RangeHandler.payload)
    r = hrr.HTTPRangeReader(range_server + "/a.zip", expected_size=size, chunk_bytes=2048, cache_chunks=3, backoff_seconds=0.01)
    with zipfile.ZipFile(r) as z:
        assert z.read("m4.bin") == bytes([4]) * 5000
    assert 0 < r.range_response_bytes < size and r.cache_hits > 0
    r.seek(-10, io.SEEK_END)
    assert r.read() == _RangeHandler.payload[-10:] and r.read(5) == b""
    assert r.seek(3) == 3 and r.read(4) == _RangeHandler.payload[3:7]


def test_http_range_reader_rejects_bad_servers_and_retries(range_server):
    size = len(_RangeHandler.payload)
    with pytest.raises(OSError, match="recorded size"):
        hrr.HTTPRangeReader(range_server + "/a.zip", expected_size=size + 1, backoff_seconds=0.01)
    with pytest.raises(OSError, match="ignored the Range"):
        hrr.HTTPRangeReader(range_server + "/norange", expected_size=size, backoff_seconds=0.01)
    _RangeHandler.fail_first = 2
    r = hrr.HTTPRangeReader(range_server + "/a.zip", expected_size=size, backoff_seconds=0.01)
    assert r.read(4) == _RangeHandler.payload[:4]
    for bad in (None, "bytes 5-2/10", "bytes 0-10/10", "items 0-1/2"):
        with pytest.raises(ValueError):
            hrr.parse_content_range(bad)
    assert hrr.parse_content_range("bytes 0-0/10") == (0, 0, 10)


def test_reference_text_scores():
    assert rq.token_f1("The cat sat.", "the CAT sat") == 1.0
    assert rq.token_f1("", "") == 1.0 and rq.token_f1("a", "") == 0.0
    assert abs(rq.token_f1("a b c d", "a b x y") - 0.5) < 1e-9
    assert rq.lcs_length("a b c d e".split(), "a x c y e".split()) == 3
    assert abs(rq.rouge_l_f1("a b c d e", "a x c y e") - 0.6) < 1e-9
    out = rq.score_reference_batch({"1": "red car", "2": "blue"}, {"1": ["a red car", "red car"], "2": ["green"]})
    assert out["samples"]["1"]["exact_match"] == 1.0 and out["mean"]["exact_match"] == 0.5
    with pytest.raises(ValueError):
        rq.score_reference_batch({"1": "x"}, {"2": ["x"]})


def test_quality_protocol_validator():
    rev = "0123456789abcdef0123456789abcdef01234567"
    good = {"schema_version": 2, "name": "p", "model": {"revision": rev, "processor_revision": rev},
            "selection": {"algorithm": "sha256-rank", "seed": 7, "materialization_requires_media_sha256": True},
            "datasets": [{"id": "docvqa", "category": "doc", "source": "hf", "repository": "x/y", "split": "val",
                          "sample_id_field": "id", "metric": "anls", "revision": rev, "development_samples": 10,
                          "final_samples": 100, "materialization_status": "materialized"}]}
    qp.validate_quality_protocol(good)
    for mutate, msg in ((lambda p: p["model"].update(revision="ABC"), "hexadecimal"),
                        (lambda p: p["datasets"].append(dict(p["datasets"][0])), "duplicate"),
                        (lambda p: p["datasets"][0].update(development_samples=1000), "exceeds"),
                        (lambda p: p["selection"].update(seed=True), "positive integer"),
                        (lambda p: p["datasets"][0].update(materialization_status="??"), "unsupported")):
        import copy
        bad = copy.deepcopy(good)
        mutate(bad)
        with pytest.raises(ValueError, match=msg):
            qp.validate_quality_protocol(bad)


def test_selection_materialisation_and_verification(tmp_path):
    import io

    from PIL import Image

    from prism_infer_b200.analysis import quality_materialization as qm
    from prism_infer_b200.utils import verify_quality_data as vq

    ids = [f"s{i}" for i in range(40)] + [7]
    sel = qm.select_sample_ids(ids, dataset_id="docvqa", revision="abc", seed=11, development_samples=5, final_samples=12)
    assert sel.final_ids[:5] == sel.development_ids and len(set(sel.final_ids)) == 12
    again = qm.select_sample_ids(list(reversed(ids)), dataset_id="docvqa", revision="abc", seed=11, development_samples=5, final_samples=12)
    assert again == sel                                    # independent of input order
    assert qm.select_sample_ids(ids, dataset_id="docvqa", revision="abc", seed=12, development_samples=5, final_samples=12) != sel
    with pytest.raises(ValueError):
        qm.select_sample_ids(["a", "a"], dataset_id="d", revision="r", seed=1, development_samples=1, final_samples=1)
    rng = np.random.default_rng(0)
    records = []
    for sid in sel.final_ids:
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, (12, 16, 3), dtype=np.uint8)).save(buf, format="PNG")
        media = qm.materialize_image(buf.getvalue(), root=tmp_path, dataset_id="docvqa")
        assert media["width"] == 16 and media["height"] == 12 and (tmp_path / media["materialized_path"]).exists()
        records.append({"sample_id": sid, "question": "q", "media": [media]})
    manifest = qm.materialization_manifest(dataset_id="docvqa", revision="abc", seed=11, selection=sel, records=records)
    out = vq.verify(manifest, records, ids, str(tmp_path))
    assert out == {"records": 12, "unique_media_files": 12, "bytes": out["bytes"]} and out["bytes"] > 0
    victim = tmp_path / records[3]["media"][0]["materialized_path"]
    victim.write_bytes(victim.read_bytes() + b"x")
    with pytest.raises(OSError, match="hash mismatch"):
        vq.verify(manifest, records, ids, str(tmp_path))
    with pytest.raises(ValueError, match="escapes"):
        qm.safe_materialized_path(tmp_path, "../x")
    with pytest.raises(ValueError, match="do not match"):
        qm.validate_selected_records(records[1:], sel.final_ids)


def test_media_groups_and_media_first_prompt():
    from prism_infer_b200.analysis import working_set_quality as wq

    def rec(sid, digests, **kw):
        return {"sample_id": sid, "media": [{"sha256": d * 64} for d in digests], **kw}

    records = [rec("a", "12"), rec("b", "21"), rec("c", "12"), rec("d", "3"), rec("e", "12"), rec("f", "21")]
    groups = wq.select_multi_question_groups(records)
    by_group = {}
    for g in groups:
        by_group.setdefault(g.media_group_id, []).append((g.record["sample_id"], g.question_index, g.group_size))
    assert sorted(by_group.values()) == [[("a", 0, 3), ("c", 1, 3), ("e", 2, 3)], [("b", 0, 2), ("f", 1, 2)]]
    assert len(wq.select_multi_question_groups(records, max_groups=1)) in (2, 3)
    assert wq.media_group_id(rec("x", "12")) != wq.media_group_id(rec("x", "12", temporal_bound={"start": 0, "end": 2}))
    with pytest.raises(ValueError):
        wq.ordered_media_sha256({"media": [{"sha256": "zz"}]})
    prompt = wq.build_media_first_prompt("Is <image> brighter than <image>?", 2, options=["A. yes", "B. no"], hint="Answer with a letter.")
    assert prompt.startswith("Image 1: <image>\nImage 2: <image>\nThe images above are numbered Image 1 through Image 2 in order.\n")
    assert "Is Image 1 brighter than Image 2?" in prompt and prompt.endswith("Answer with a letter.")
    dense = [{"sample_id": i, "correct": i % 2 == 0} for i in range(6)]
    compact = [{"sample_id": i, "correct": i % 3 == 0, "deleted_visual_tokens": 10 if i >= 2 else 0} for i in range(6)]
    assert wq.paired_deleted_subset(dense, compact) == {"cohort": 4, "dense_correct": 2, "compact_correct": 1}
    assert wq.summarize_stage_samples(compact)["samples_with_deletions"] == 4


def test_materialize_quality_subset_from_local_parquet_shards(tmp_path):
    """Two complete shards of a MuirBench-like dataset and one DocVQA-like shard, written with
    pyarrow: selection is deterministic, only the selected rows are materialised, the manifest
    verifies, an incomplete shard set is refused."""
    import io
    import json

    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq
    import pytest
    from PIL import Image

    from prism_infer_b200.analysis import quality_materialization as qmat
    from prism_infer_b200.utils import materialize_quality_data as mq

    rng = np.random.default_rng(0)

    def png():
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, (24, 24, 3), dtype=np.uint8)).save(buf, format="PNG")
        return {"bytes": buf.getvalue(), "path": None}

    shared = png()
    raw = tmp_path / "raw"
    raw.mkdir()
    rows = [{"idx": i, "task": "t", "image_relation": "r", "image_type": "photo", "question": f"q{i} <image> <image>", "options": ["a", "b", "c"],
             "answer": "ABC"[i % 3], "image_list": [shared, png()], "counterpart_idx": -1} for i in range(10)]
    pq.write_table(pa.Table.from_pylist(rows[:6]), raw / "test-00000-of-00002.parquet")
    pq.write_table(pa.Table.from_pylist(rows[6:]), raw / "test-00001-of-00002.parquet")
    out = tmp_path / "quality"
    m = mq.materialize(layout="muirbench", dataset_id="muir", revision="rev1", raw_dir=raw, split="test", out_root=out, seed=7,
                       development=2, final=4, batch_size=3)
    assert m["selection"]["population_samples"] == 10 and m["selection"]["final"]["samples"] == 4 and len(m["source_files"]) == 2
    records = [json.loads(line) for line in (out / "muir.records.jsonl").read_text().splitlines()]
    assert [r["sample_id"] for r in records] == m["selection"]["final"]["sample_ids"]
    assert m["verification"]["unique_media_files"] == 5                      # 4 private images + the shared one, stored once
    assert len({r["media"][0]["sha256"] for r in records}) == 1
    qmat.verify_materialized_records(records, out)
    # the stand-alone verifier reproduces the selection from the population list written beside the manifest
    from prism_infer_b200.utils import verify_quality_data as vq

    report = vq.verify(json.loads((out / "muir.manifest.json").read_text()), records, json.loads((out / "muir.population.json").read_text()), str(out))
    assert report
    with pytest.raises(ValueError):
        vq.verify(json.loads((out / "muir.manifest.json").read_text()), records, ["0", "1", "2", "3", "4"], str(out))
    again = mq.materialize(layout="muirbench", dataset_id="muir", revision="rev1", raw_dir=raw, split="test", out_root=out, seed=7,
                           development=2, final=4)
    assert again["records_sha256"] == m["records_sha256"]                    # idempotent
    other = mq.materialize(layout="muirbench", dataset_id="muir", revision="rev2", raw_dir=raw, split="test", out_root=tmp_path / "q2", seed=7,
                           development=2, final=4)
    assert other["selection"]["final"]["sample_ids"] != m["selection"]["final"]["sample_ids"]   # the revision is part of the preimage
    (raw / "test-00001-of-00002.parquet").unlink()
    with pytest.raises(ValueError, match="incomplete"):
        mq.discover_complete_shards(raw, "test")
    with pytest.raises(FileNotFoundError):
        mq.discover_complete_shards(raw, "validation")

    doc = tmp_path / "doc"
    doc.mkdir()
    drows = [{"questionId": 100 + i, "question": f"what {i}", "answers": ["x", "y"], "image": png(), "question_types": ["form"], "docId": i}
             for i in range(5)]
    pq.write_table(pa.Table.from_pylist(drows), doc / "validation-00000-of-00001.parquet")
    dm = mq.materialize(layout="docvqa", dataset_id="docvqa", revision="r", raw_dir=doc, split="validation", out_root=out, seed=1,
                        development=1, final=3)
    drec = [json.loads(line) for line in (out / "docvqa.records.jsonl").read_text().splitlines()]
    assert len(drec) == 3 and drec[0]["answers"] == ["x", "y"] and dm["layout"] == "docvqa"
    with pytest.raises(ValueError, match="outside its options"):
        mq.convert_row("muirbench", dict(rows[0], answer="D"), root=out, dataset_id="muir")
    with pytest.raises(ValueError, match="no embedded image"):
        mq.convert_row("docvqa", dict(drows[0], image={"path": "x.png"}), root=out, dataset_id="docvqa")
