"""Working-set matrix runner (resume logic) and summariser, on fabricated cell records (CPU)."""

import importlib.util
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "benchmarks", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _record(ttft):
    from prism_infer_b200.analysis import benchmark_schema

    return {"schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "online_working_set", "engine": "prism_infer_b200",
            "model": "random:tiny", "data": "synthetic", "hardware": {"gpus": 1}, "config": {"variant": "compact_prefix"},
            "results": {"ttft_p50_ms": ttft, "ttft_p99_ms": ttft * 2, "e2e_p50_ms": 80.0, "e2e_p99_ms": 120.0,
                        "recomputed_prompt_tokens": 100, "output_tokens_per_s": 64.0, "resident_media": 42, "prefix_evictions": 0}}


def test_matrix_resume_skips_complete_cells_and_archives_interrupted_ones(tmp_path):
    m = _load("run_working_set_matrix")
    out = str(tmp_path)
    assert len(m.plan_cells(out, resume=True, only=[])) == 9
    done = os.path.join(out, m.cell_name("fit", "compact_prefix") + ".json")
    with open(done, "w") as fh:
        json.dump(_record(11.0), fh)
    broken = os.path.join(out, m.cell_name("knee", "dense_prefix") + ".json")
    with open(broken, "w") as fh:
        fh.write("{\"schema_version\": 1")                     # interrupted write
    with open(os.path.join(out, m.cell_name("pressure", "vision_only") + ".json.tmp"), "w") as fh:
        fh.write("{}")
    todo = m.plan_cells(out, resume=True, only=[])
    names = {m.cell_name(w, v) for w, v, _ in todo}
    assert len(todo) == 8 and "fit__compact_prefix" not in names and "knee__dense_prefix" in names
    assert os.path.exists(done) and not os.path.exists(broken)
    assert len(os.listdir(os.path.join(out, "interrupted"))) == 2
    assert len(m.plan_cells(out, resume=False, only=["fit"])) == 3   # without --resume a finished cell runs again
    assert not os.path.exists(done)


def test_summary_table(tmp_path):
    s = _load("summarize_working_set")
    for name, ttft in (("fit__compact_prefix", 11.0), ("pressure__dense_prefix", 18.0)):
        with open(tmp_path / f"{name}.json", "w") as fh:
            json.dump(_record(ttft), fh)
    rows = s.summary_rows(s.load_cells(str(tmp_path)))
    assert [r["working_set"] for r in rows] == ["fit", "pressure"] and rows[1]["variant"] == "dense_prefix"
    assert rows[0]["ttft_p99_ms"] == 22.0
    table = s.to_markdown(rows)
    assert table.count("\n") == 3 and "| pressure | dense_prefix | 18.0 | 36.0 |" in table


def test_working_set_plan_builder_measures_resumes_and_round_trips(tmp_path):
    """Dense prefix pages measured on the tiny model, an interrupted run resumed, a foreign page
    artifact refused, the plan document reloaded and protected against edits."""
    import pytest
    import torch

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import working_set_plan as wsp
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    b = _load("build_working_set_plan")
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    groups = wsp.synthetic_groups(4, 9, seed=3, min_images=1, max_images=3, tokens_per_image=6, page=16, question_tokens=(3, 6))
    groups = [wsp.MediaGroup(g.group_id, g.media_digests, tuple(" ".join(str(int(t) % 900 + 10) for t in q.split()) for q in g.questions),
                             g.dense_prefix_pages) for g in groups]
    contract = b.measurement_contract(model="random:tiny", page_tokens=16, image_size=64, seed=3, groups=groups)
    engines = []

    def make_engine():
        engines.append(LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=128,
                           enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=True))
        return engines[-1]

    art_path = tmp_path / "plan.json.pages.json"
    lines = []
    first = b.measure_all(groups[:2], art_path, contract, make_engine, 64, resume=False, log=lines.append)
    assert len(first["groups"]) == 2 and len(lines) == 2 and len(engines) == 1
    with pytest.raises(FileExistsError):
        b.measure_all(groups, art_path, contract, make_engine, 64, resume=False)
    full = b.measure_all(groups, art_path, contract, make_engine, 64, resume=True, log=lines.append)
    assert len(full["groups"]) == 4 and len(lines) == 4 and len(engines) == 2      # only the two missing groups ran
    again = b.measure_all(groups, art_path, contract, make_engine, 64, resume=True)
    assert again == full and len(engines) == 2                                     # nothing left: no engine built
    for g in groups:  # a 64x64 image is 4 visual tokens; pages of 16 tokens
        m = full["groups"][g.group_id]
        assert m["images"] == g.num_images and m["dense_prefix_pages"] == -(-m["prefix_tokens"] // 16) >= 1
    other = dict(contract, image_size=128)
    with pytest.raises(ValueError, match="different contract"):
        b.measure_all(groups, art_path, other, make_engine, 64, resume=True)

    measured = [wsp.MediaGroup(g.group_id, g.media_digests, g.questions, full["groups"][g.group_id]["dense_prefix_pages"]) for g in groups]
    plan = wsp.build_plan(wsp.select_groups(measured, 4, "all"), num_requests=12, rate=50.0, seed=3, page_budget=4)
    doc = b.plan_document(plan, contract, "all")
    path = tmp_path / "plan.json"
    path.write_text(json.dumps(doc))
    loaded, doc2 = b.load_plan_document(path)
    assert doc2["plan_sha256"] == doc["plan_sha256"] and loaded.measured == plan.measured and loaded.groups == plan.groups
    doc["page_budget"] = 999
    path.write_text(json.dumps(doc))
    with pytest.raises(ValueError, match="edited"):
        b.load_plan_document(path)
