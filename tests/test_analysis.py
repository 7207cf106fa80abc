"""Analysis helpers: percentiles, online summaries, working-set plans, schemas, quality metrics."""

import json

import pytest

from prism_infer_b200.analysis import benchmark_schema as bs
from prism_infer_b200.analysis import online_serving as osv
from prism_infer_b200.analysis import performance_profile as pp
from prism_infer_b200.analysis import quality_metrics as qm
from prism_infer_b200.analysis import working_set_plan as wsp
from prism_infer_b200.analysis.identity import record_identity
from prism_infer_b200.observability import profile_region
from prism_infer_b200.runtime_capabilities import probe_runtime_capabilities, validate_runtime_capabilities


def test_percentile_is_linear_interpolation():
    assert osv.percentile([10, 20, 30, 40], 0.5) == 25.0
    assert osv.percentile([1, 2, 3], 0.99) == pytest.approx(2.98)
    assert osv.percentile([5], 0.9) == 5
    with pytest.raises(ValueError):
        osv.percentile([], 0.5)
    with pytest.raises(ValueError):
        osv.percentile([1.0, float("nan")], 0.5)


def test_online_summary_counts_recomputed_tokens():
    reqs = [
        {"finish_reason": "length", "ttft_ms": 100.0, "latency_ms": 300.0, "prompt_tokens": 500, "cached_tokens": 400, "token_ids": [1] * 16},
        {"finish_reason": "length", "ttft_ms": 200.0, "latency_ms": 500.0, "prompt_tokens": 300, "cached_tokens": 0, "token_ids": [1] * 16},
        {"finish_reason": "cancelled", "prompt_tokens": 50, "cached_tokens": 0, "token_ids": []},
    ]
    s = osv.summarize_online_run({"duration_s": 2.0, "requests": reqs})
    assert s["requests"] == {"total": 3, "completed": 2, "rejected": 0, "cancelled": 1}
    assert s["recomputed_prompt_tokens"] == 400 and s["output_tokens_per_s"] == 16.0
    assert s["ttft_ms"]["p50"] == 150.0
    with pytest.raises(ValueError):
        osv.summarize_online_run({"duration_s": 1.0, "requests": [{"finish_reason": None}]})


def test_working_set_plan_is_deterministic_and_follows_the_definitions():
    groups = wsp.synthetic_groups()
    assert len(groups) == 42 and sum(len(g.questions) for g in groups) == 85
    assert all(1 <= g.num_images <= 8 and 2 <= len(g.questions) <= 3 for g in groups)
    plan = wsp.build_plan(groups)
    again = wsp.build_plan(wsp.synthetic_groups())
    assert plan.to_record() == again.to_record()
    assert len(plan.population) == 42 and all(r.question_index == 0 for r in plan.population)
    assert len(plan.measured) == 600
    offsets = [r.arrival_offset_s for r in plan.measured]
    assert offsets == sorted(offsets) and 120 < offsets[-1] < 180  # Poisson at 4 req/s
    # every measured request asks a different question than the group's previous request
    last = {i: 0 for i in range(42)}
    for r in plan.measured:
        assert r.question_index != last[r.group_index]
        last[r.group_index] = r.question_index
    counts = [sum(1 for r in plan.measured if r.group_index == g) for g in range(42)]
    assert counts[0] > counts[10] > 0  # Zipf: low ranks dominate
    assert [g.group_id for g in plan.groups] == sorted(g.group_id for g in groups)
    fit = wsp.select_groups(groups, 100, "fit")
    knee = wsp.select_groups(groups, 100, "knee")
    pressure = wsp.select_groups(groups, 100, "pressure")
    assert sum(g.dense_prefix_pages for g in fit) <= 70 < 100 < sum(g.dense_prefix_pages for g in knee)
    assert sum(g.dense_prefix_pages for g in pressure) >= 148
    assert wsp.media_first_prompt(2, "Q?").startswith("Image 1: <image>\nImage 2: <image>\n")
    assert wsp.media_first_prompt(2, "Q?").endswith("in order.\nQ?")


def test_benchmark_schema_validation_and_no_overwrite(tmp_path):
    rec = {"schema_version": 1, "benchmark": "decode", "engine": "prism_b200", "model": "tiny", "hardware": {"gpu": "B200"},
           "data": "synthetic", "config": {"batch": 1}, "results": {"tpot_ms": 4.6, "tok_per_s": 217.0}}
    bs.validate_benchmark_record(rec)
    path = tmp_path / "r.json"
    bs.write_record(str(path), rec)
    assert json.loads(path.read_text())["results"]["tpot_ms"] == 4.6
    with pytest.raises(FileExistsError):
        bs.write_record(str(path), rec)
    bad = dict(rec, results={"tpot_ms": float("inf")})
    with pytest.raises(bs.SchemaError):
        bs.validate_benchmark_record(bad)
    with pytest.raises(bs.SchemaError):
        bs.validate_benchmark_record({k: v for k, v in rec.items() if k != "hardware"})
    with pytest.raises(bs.SchemaError):
        bs.validate_benchmark_record(dict(rec, results={"tpot_ms": -1.0}))
    assert record_identity({"a": 1, "b": 2}) == record_identity({"b": 2, "a": 1})


def test_quality_metrics():
    assert qm.anls("The Cat", ["the cat", "dog"]) == 1.0
    assert qm.anls("kitten", ["sitting"]) == pytest.approx(1 - 3 / 7)
    assert qm.anls("completely different", ["x"]) == 0.0
    assert qm.parse_choice("The answer is (B).") == "B" and qm.parse_choice("C") == "C"
    assert qm.parse_choice("maybe E", num_options=4) is None
    assert qm.choice_accuracy(["A", "(B)", "none"], ["A", "B", "C"]) == pytest.approx(2 / 3)


def test_profile_session_records_regions_and_is_noop_outside():
    with profile_region("outside"):
        pass
    with pp.performance_profile({"run": "t"}, cuda_timing=False, nvtx=False) as session:
        with profile_region("a.b", cuda=False, metadata={"k": 1}):
            with profile_region("inner", cuda=False):
                pass
        with profile_region("a.b", cuda=False):
            pass
    rec = pp.validate_profile_record(session.finalize())
    assert rec["totals"]["a.b"]["count"] == 2 and rec["totals"]["inner"]["count"] == 1
    # regions are listed in start order, each with the index of its enclosing region
    assert [r["name"] for r in rec["regions"]] == ["a.b", "inner", "a.b"] and rec["metadata"] == {"run": "t"}
    assert [r["parent"] for r in rec["regions"]] == [None, 0, None]
    assert rec["regions"][0]["start_ns"] <= rec["regions"][1]["start_ns"] <= rec["regions"][2]["start_ns"]
    with profile_region("after"):
        pass
    assert len(session.regions) == 3


def test_runtime_capabilities_fail_closed():
    rep = probe_runtime_capabilities(require_cuda=False)
    assert rep.torch_version and rep.fp8_dtype
    import torch

    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            validate_runtime_capabilities(require_cuda=True)
