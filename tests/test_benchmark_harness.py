"""Shared benchmark harness: source / GPU identity, case manifests, exact content-reuse
workloads, the process-memory sampler against a fake NVML, and the media-cache benchmark on the
tiny model (CPU)."""

import importlib.util
import json
import os
import sys
import time

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
    try:
        spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "benchmarks", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod
    finally:
        sys.path.pop(0)


def test_source_identity_tracks_content(tmp_path):
    h = _load("harness")
    (tmp_path / "prism_infer_b200").mkdir()
    (tmp_path / "prism_infer_b200" / "a.py").write_text("x = 1\n")
    (tmp_path / "prism_infer_b200" / "notes.txt").write_text("ignored")
    (tmp_path / "bench.py").write_text("pass\n")
    d1, n1 = h.source_tree_sha256(tmp_path)
    assert n1 == 2
    (tmp_path / "prism_infer_b200" / "notes.txt").write_text("still ignored")
    assert h.source_tree_sha256(tmp_path) == (d1, 2)
    (tmp_path / "prism_infer_b200" / "a.py").write_text("x = 2\n")
    assert h.source_tree_sha256(tmp_path)[0] != d1
    ident = h.collect_source_identity(tmp_path)     # not a checkout: commit and dirty unknown, digest present
    assert ident.commit is None and ident.dirty is None and len(ident.tree_sha256) == 64
    here = h.collect_source_identity()
    assert here.files > 50 and here.to_record()["tree_sha256"] == h.source_tree_sha256()[0]


def test_gpu_query_parsing():
    h = _load("harness")
    rows = h.parse_gpu_query("0, NVIDIA B200, GPU-abc, 580.159, 183359, 1965, 3996, 1000.00\n1, NVIDIA B200, GPU-def, 580.159, 183359, 1965, 3996, [N/A]\n")
    assert rows[0].uuid == "GPU-abc" and rows[0].sm_max_mhz == 1965.0 and rows[1].power_limit_w is None and rows[1].index == 1
    with pytest.raises(ValueError):
        h.parse_gpu_query("0, only, three")
    prov = h.provenance()
    assert "source" in prov and "gpu" in prov   # gpu is None on a machine without one


def test_manifest_cases_expand_and_materialize():
    h = _load("harness")
    manifest = json.load(open(os.path.join(ROOT, "benchmarks", "workloads", "system_cases.json")))
    case = h.find_workload_case(manifest, "mixed_text_image_video")
    with pytest.raises(ValueError, match="available cases"):
        h.find_workload_case(manifest, "nope")
    expanded, source, factor = h.expand_case_batch(case, 6)
    assert (source, factor, len(expanded["requests"])) == (3, 2, 6) and len(case["requests"]) == 3
    for bad in (2, 4, 0):
        with pytest.raises(ValueError):
            h.expand_case_batch(case, bad)
    payloads = h.materialize_requests(expanded)
    assert [p["type"] for p in payloads] == ["text", "image", "video"] * 2
    assert payloads[1]["image"].shape == (448, 448, 3) and len(payloads[2]["video"]) == 4
    assert np.array_equal(payloads[1]["image"], payloads[4]["image"])      # seeded: the same pixels every time
    flat = h.make_image({"width": 4, "height": 2, "color": [1, 2, 3]})
    assert flat.shape == (2, 4, 3) and (flat == np.array([1, 2, 3], dtype=np.uint8)).all()
    d = h.describe_case_inputs(case)
    assert (d["images"], d["videos"], d["video_frames"]) == (1, 1, 4) and d["input_shapes"][0]["visual_shapes"] == []
    for c in manifest["cases"]:
        h.materialize_requests({"requests": [dict(r, **({"image": dict(r["image"], width=32, height=32)} if "image" in r else {})) for r in c["requests"]
                                             if r["type"] in ("text", "image")]})


@pytest.mark.parametrize("rate,repeats", [(0.0, 0), (0.5, 3), (1.0, 6), (0.34, 2)])
def test_content_reuse_workload_has_exact_repeat_count(rate, repeats):
    h = _load("harness")
    img = np.random.default_rng(0).integers(0, 256, (32, 32, 3), dtype=np.uint8)
    base = [{"type": "text", "prompt": "t"}] + [{"type": "image", "prompt": "q", "image": img} for _ in range(4)] + \
           [{"type": "video", "prompt": "v", "video": [img, img]} for _ in range(2)]
    out, info = h.build_multimodal_cache_workload(base, repeat_rate=rate, vary_questions=True)
    assert info["media_requests"] == 6 and info["repeated_media_requests"] == repeats and info["unique_media_requests"] == 6 - repeats
    media = [p.get("image") if "image" in p else p["video"][0] for p in out[1:]]
    same = [np.array_equal(m, img) for m in media]
    assert sum(same) == repeats
    assert all(m is not img for m in media)                               # fresh arrays, identical or not
    distinct = {m.tobytes() for m, s in zip(media, same) if not s}
    assert len(distinct) == 6 - repeats                                   # every unique request differs from all others
    assert out[0] == base[0] and out[1]["prompt"].endswith("variant 1 concisely.")
    assert np.array_equal(out[-1]["video"][1], img)                        # only the first frame carries the marker
    with pytest.raises(ValueError):
        h.build_multimodal_cache_workload(base, repeat_rate=1.5, vary_questions=False)


def test_memory_sampler_with_fake_nvml():
    h = _load("harness")

    class Proc:
        def __init__(self, pid, used):
            self.pid, self.usedGpuMemory = pid, used

    class FakeNvml:
        calls = 0
        shut = False

        def nvmlInit(self): ...
        def nvmlDeviceGetHandleByIndex(self, i): return ("handle", i)
        def nvmlShutdown(self): FakeNvml.shut = True

        def nvmlDeviceGetComputeRunningProcesses(self, handle):
            FakeNvml.calls += 1
            return [Proc(4242, 100 * FakeNvml.calls if FakeNvml.calls < 4 else 50), Proc(1, 10 ** 12), Proc(4242, None)]

    with h.GpuMemorySampler(0, pid=4242, period_s=0.001, nvml=FakeNvml()) as s:
        t0 = time.time()
        while s.samples < 6 and time.time() - t0 < 5:
            time.sleep(0.002)
    rec = s.to_record()
    assert rec["peak_bytes"] == 300 and rec["last_bytes"] == 50 and rec["samples"] >= 6 and rec["error"] is None and FakeNvml.shut

    class Broken(FakeNvml):
        def nvmlInit(self): raise RuntimeError("no driver")

    with h.GpuMemorySampler(0, nvml=Broken()) as s:
        time.sleep(0.01)
    assert "no driver" in s.to_record()["error"] and s.peak_bytes == 0


def test_media_cache_benchmark_on_tiny_model():
    import torch

    from prism_infer_b200 import LLM
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    _load("harness")
    b = _load("bench_media_cache")
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    llm = LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=256, enforce_eager=True,
              max_num_batched_tokens=512, max_chunk_size=512, max_num_seqs=8, enable_prefix_caching=True, enable_visual_embedding_cache=True)
    case = {"id": "tiny_image", "requests": [{"type": "image", "prompt": [5, 6, 7, 8], "image": {"width": 64, "height": 64, "seed": 9}}]}
    try:
        cells = b.run_rates(llm, case, 4, [0.0, 1.0], vary_questions=False, max_tokens=2, nvml=object())
    finally:
        llm.exit()
    unique, repeated = cells
    assert unique["requests"] == 4 and unique["reuse"]["repeated_media_requests"] == 0 and unique["output_tokens"] == 8
    # every unique image is encoded once (a miss at submission; the prefill then reads the stored embedding)
    assert unique["visual_embedding_cache"]["misses"] == 4 and unique["prefix_cache"]["hits"] == 0
    assert repeated["reuse"]["repeated_media_requests"] == 4
    assert repeated["visual_embedding_cache"]["misses"] <= 1                                   # at most the first request encodes
    assert repeated["process_gpu_memory"]["error"] is not None                                 # the fake NVML has no methods: recorded, not raised


def test_workload_manifest_contract_and_file_images(tmp_path):
    """The shipped manifest is valid; every kind of defect is named; an image_file request is read with its hash
    and size checked; a caption task's references are scored against a prediction."""
    import copy
    import hashlib
    import io

    import numpy as np
    import pytest
    from PIL import Image

    from prism_infer_b200.analysis import workload_manifest as wm
    from prism_infer_b200.analysis.reference_quality import score_reference_text

    h = _load("harness")
    shipped = h.load_manifest(os.path.join(ROOT, "benchmarks", "workloads", "system_cases.json"))
    assert {c["id"] for c in shipped["cases"]} >= {"text_short", "single_image_448", "mixed_text_image_video"}

    buf = io.BytesIO()
    Image.fromarray(np.random.default_rng(0).integers(0, 256, (48, 64, 3), dtype=np.uint8)).save(buf, format="PNG")
    (tmp_path / "media").mkdir()
    (tmp_path / "media" / "cat.png").write_bytes(buf.getvalue())
    digest = hashlib.sha256(buf.getvalue()).hexdigest()
    manifest = {
        "schema_version": 1, "name": "captioning",
        "reference_sources": {"coco": {"dataset": "COCO", "split": "val2017", "task": "caption", "source_url": "https://example.org/coco",
                                       "annotation_file": "captions_val2017.json", "content_sha256": "ab" * 32}},
        "cases": [{"id": "one_caption", "requests": [
            {"type": "image_file", "prompt": "Describe the image.",
             "image": {"path": "media/cat.png", "source_url": "https://example.org/cat.png", "sha256": digest, "width": 64, "height": 48},
             "evaluation": {"task": "caption", "reference_source": "coco", "image_id": 7,
                            "references": [{"annotation_id": 1, "text": "A cat sits on a mat."}, {"annotation_id": 2, "text": "a small cat resting"}]}},
            {"type": "interleaved_images", "prompt": "<image> and <image>", "images": [{"width": 32, "height": 32, "seed": 1},
                                                                                    {"width": 32, "height": 32, "color": [1, 2, 3]}]},
            {"type": "video", "prompt": "what moves", "frames": [{"width": 32, "height": 32, "seed": 2}, {"width": 32, "height": 32, "seed": 3}]},
        ]}],
    }
    path = tmp_path / "m.json"
    path.write_text(json.dumps(manifest))
    loaded = h.load_manifest(path)
    case = h.find_workload_case(loaded, "one_caption")
    payloads = h.materialize_requests(case, base=tmp_path)
    assert payloads[0]["type"] == "image" and payloads[0]["image"].shape == (48, 64, 3)
    assert h.describe_case_inputs(case)["images"] == 3 and h.describe_case_inputs(case)["video_frames"] == 2
    refs = [r["text"] for r in case["requests"][0]["evaluation"]["references"]]
    assert score_reference_text("a cat sits on a mat", refs)["token_f1"] == 1.0
    with pytest.raises(ValueError, match="needs the manifest's directory"):
        h.materialize_requests(case)
    (tmp_path / "media" / "cat.png").write_bytes(buf.getvalue() + b"x")
    with pytest.raises(ValueError, match="sha256"):
        h.materialize_requests(case, base=tmp_path)

    def broken(mutate, needle):
        bad = copy.deepcopy(manifest)
        mutate(bad)
        with pytest.raises(wm.ManifestError, match=needle):
            wm.validate_workload_manifest(bad)

    req = lambda m, i: m["cases"][0]["requests"][i]  # noqa: E731
    broken(lambda m: m.update(schema_version=2), "schema_version")
    broken(lambda m: m["cases"].append(copy.deepcopy(m["cases"][0])), "appears twice")
    broken(lambda m: m["cases"][0].update(requests=[]), "requests")
    broken(lambda m: req(m, 0).update(type="audio"), "not one of")
    broken(lambda m: req(m, 0)["image"].update(sha256="XYZ"), "sha256")
    broken(lambda m: req(m, 0)["image"].update(path="../cat.png"), "below the manifest")
    broken(lambda m: req(m, 0)["evaluation"].update(reference_source="flickr"), "unknown source")
    broken(lambda m: req(m, 0)["evaluation"].update(task="free_text_qa"), "is a 'caption' source")
    broken(lambda m: req(m, 0)["evaluation"]["references"].append({"annotation_id": 1, "text": "again"}), "twice")
    broken(lambda m: req(m, 0)["evaluation"]["references"][0].update(text="?!"), "no word left")
    broken(lambda m: req(m, 1).update(prompt="<image> only"), "markers for 2 images")
    broken(lambda m: req(m, 1)["images"][0].update(color=[0, 0, 0]), "exactly one of")
    broken(lambda m: req(m, 1)["images"][1].update(color=[0, 0, 256]), "0..255")
    broken(lambda m: req(m, 2)["frames"][1].update(width=16), "same size")
    broken(lambda m: req(m, 2).update(frames=[]), "frames")
    broken(lambda m: m["reference_sources"]["coco"].pop("split"), "split is missing")
