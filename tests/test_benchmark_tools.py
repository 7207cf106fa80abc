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
