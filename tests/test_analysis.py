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
    assert all(r["step_id"] is None and r["phase"] == "preprocess" for r in rec["regions"])
    assert rec["summary"]["a.b"]["calls"] == 2 and rec["summary"]["a.b"]["cuda_ms"] is None
    assert set(rec["summary"]["a.b"]["cpu_ms"]) == set(pp.STAT_KEYS) and set(rec["summary_by_phase"]) == {"preprocess"}


def test_profile_of_engine_steps_links_regions_to_steps_and_phases():
    """An engine run inside a session: every ``engine.step`` region opens a step, the regions below it carry its id
    and phase, the summaries split by phase, and a doctored aggregate is refused."""
    import copy

    import torch

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    arch = Qwen3VLArch.tiny()
    llm = LLM("random:tiny", weights=random_weights(arch, dtype=torch.float32, seed=0), device="cpu", max_model_len=128,
              kvcache_block_size=16, num_kvcache_blocks=16, enforce_eager=True)
    with pp.performance_profile({"run": "engine"}, cuda_timing=False, nvtx=False) as session:
        with profile_region("submit", cuda=False):
            llm.add_request([5, 6, 7, 8], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
        while not llm.is_finished():
            llm.step_result()
    llm.exit()
    rec = pp.validate_profile_record(session.finalize())
    assert [s["phase"] for s in rec["steps"]] == ["prefill", "decode", "decode"] and [s["step_id"] for s in rec["steps"]] == [0, 1, 2]
    assert all(s["status"] == "ok" and s["batch_size"] == 1 for s in rec["steps"])
    by_name = {}
    for r in rec["regions"]:
        by_name.setdefault(r["name"], []).append(r)
    assert [r["step_id"] for r in by_name["engine.step"]] == [0, 1, 2]
    assert by_name["submit"][0]["phase"] == "preprocess" and by_name["submit"][0]["step_id"] is None
    assert {r["phase"] for r in by_name["engine.scheduler.schedule"]} == {"prefill", "decode"}
    assert set(rec["summary_by_phase"]) == {"preprocess", "prefill", "decode"}
    assert rec["summary_by_phase"]["decode"]["engine.step"]["calls"] == 2 and rec["summary"]["engine.step"]["calls"] == 3
    stats = rec["summary"]["engine.step"]["cpu_ms"]
    assert stats["min"] <= stats["median"] <= stats["p90"] <= stats["p99"] <= stats["max"]
    for mutate, needle in (
        (lambda r: r["summary"]["engine.step"].update(calls=4), "summary does not follow"),
        (lambda r: r["regions"][2].update(phase="decode" if r["regions"][2]["phase"] != "decode" else "prefill"), "its step says"),
        (lambda r: r["regions"][1].update(step_id=9), "unknown step"),
        (lambda r: r["steps"][1].update(step_id=0), "distinct"),
        (lambda r: r["regions"][0].update(cpu_ms=-1.0), "non-negative"),
        (lambda r: r["totals"]["engine.step"].update(count=1), "totals do not follow"),
    ):
        bad = copy.deepcopy(rec)
        mutate(bad)
        with pytest.raises(ValueError, match=needle):
            pp.validate_profile_record(bad)
    # a step that raises is recorded as an error step
    with pp.performance_profile(cuda_timing=False, nvtx=False) as session:
        with pytest.raises(RuntimeError):
            with profile_region("engine.step", cuda=False):
                raise RuntimeError("boom")
    assert session.finalize()["steps"] == [{"step_id": 0, "status": "error"}]


def test_runtime_capabilities_fail_closed():
    rep = probe_runtime_capabilities(require_cuda=False)
    assert rep.torch_version and rep.fp8_dtype
    import torch

    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CUDA device"):
            validate_runtime_capabilities(require_cuda=True)


def _record(benchmark, config, results, gpus=1):
    return {"schema_version": bs.BENCHMARK_SCHEMA_VERSION, "benchmark": benchmark, "engine": "prism_infer_b200", "model": "random:tiny",
            "hardware": {"gpus": gpus}, "data": "synthetic", "config": config, "results": results}


def test_each_benchmark_has_its_own_record_contract():
    """A record must carry the fields of its benchmark and satisfy the relations between them."""
    import copy

    row = {"batch": 8, "ttft_ms_mean": 30.0, "ttft_ms_max": 45.0, "tpot_ms_mean": 3.1, "output_tok_per_s": 1800.0, "preprocess_ms": 17.0,
           "steady_step_ms_median": 3.2, "steady_tok_per_s": 2500.0}
    good = _record("decode_matrix", {"workload": "image1", "output_tokens": 64, "tp": 8, "kv": "scaled_fp8"}, {"rows": [row]}, gpus=8)
    bs.validate_benchmark_record(good)
    for mutate, needle in (
        (lambda r: r["results"]["rows"][0].pop("tpot_ms_mean"), "tpot_ms_mean is missing"),
        (lambda r: r["results"]["rows"][0].update(ttft_ms_max=10.0), "below the mean"),
        (lambda r: r["results"]["rows"][0].update(steady_tok_per_s=9000.0), "does not follow"),
        (lambda r: r["results"]["rows"].append(dict(row)), "appears twice"),
        (lambda r: r["hardware"].update(gpus=2), "disagree"),
        (lambda r: r["results"]["rows"][0].update(batch=0), "not a valid posint"),
    ):
        bad = copy.deepcopy(good)
        mutate(bad)
        with pytest.raises(bs.SchemaError, match=needle):
            bs.validate_benchmark_record(bad)

    online = _record("online_working_set",
                     {"variant": "compact", "groups": 42, "questions": 85, "requests": 600, "rate_per_s": 4.0, "pages": 220, "page_tokens": 256,
                      "kv_budget_bytes": 220 * 1000, "working_set_pages": 312, "max_tokens": 16, "tp": 1},
                     {"ttft_p50_ms": 14.2, "ttft_p99_ms": 29.3, "e2e_p50_ms": 76.6, "e2e_p99_ms": 101.7, "recomputed_prompt_tokens": 29984,
                      "prompt_tokens": 400000, "output_tokens_per_s": 63.0, "completed": 600, "duration_s": 151.0, "resident_media": 42,
                      "prefix_evictions": 0, "prefix_hits": 558, "resident_pages": 168})
    bs.validate_benchmark_record(online)
    for key, value, needle in (("ttft_p99_ms", 1.0, "below"), ("recomputed_prompt_tokens", 10 ** 9, "recomputed"), ("completed", 601, "completed"),
                               ("resident_pages", 221, "budget"), ("resident_media", 43, "groups")):
        bad = copy.deepcopy(online)
        bad["results"][key] = value
        with pytest.raises(bs.SchemaError, match=needle):
            bs.validate_benchmark_record(bad)

    cell = {"repeat_rate": 0.5, "requests": 8, "wall_s": 0.4, "requests_per_s": 20.0, "output_tokens": 64,
            "visual_embedding_cache": {"hits": 4, "misses": 4}, "prefix_cache": {"hits": 4, "misses": 4, "stores": 4, "evictions": 0}}
    media = _record("media_cache_reuse", {"case": "eight_image_448", "batch": 8, "mode": "scaled_fp8_kv", "max_tokens": 8}, {"cells": [cell]})
    bs.validate_benchmark_record(media)
    bad = copy.deepcopy(media)
    bad["results"]["cells"][0]["output_tokens"] = 65
    with pytest.raises(bs.SchemaError, match="more output tokens"):
        bs.validate_benchmark_record(bad)
    bad = copy.deepcopy(media)
    bad["results"]["cells"][0]["repeat_rate"] = 1.5
    with pytest.raises(bs.SchemaError, match="frac"):
        bs.validate_benchmark_record(bad)

    system = _record("system_mode_matrix", {"mode": "graph", "workload": "single_image_448", "tp": 1},
                     {"ttft_ms": 16.0, "tpot_ms": 3.9, "e2e_ms": 500.0, "output_tokens_per_s": 250.0, "batch": 1})
    system["schema_version"] = 2  # the four headline numbers only
    bs.validate_benchmark_record(system)
    system["results"]["e2e_ms"] = 1.0
    with pytest.raises(bs.SchemaError, match="below"):
        bs.validate_benchmark_record(system)


def _stats(values):
    v = sorted(values)
    return {"count": len(v), "median": v[len(v) // 2], "p90": v[-1], "p99": v[-1], "min": v[0], "max": v[-1]}


def _system_record():
    from prism_infer_b200.analysis.identity import canonical_json_sha256

    ids = [[5, 6, 7, 8], [9, 9, 1, 2], [3, 3, 3, 3]]
    stats = {"ttft_ms": _stats([16.0, 15.0, 17.0]), "tpot_ms": _stats([3.9, 3.8, 4.0]), "e2e_ms": _stats([500.0, 499.0, 501.0]),
             "output_tokens_per_s": _stats([24.0, 23.0, 25.0])}
    rec = _record("system_mode_matrix",
                  {"mode": "graph_visual_compact_scaled_fp8", "workload": "single_image_448", "tp": 1, "repeats": 3, "output_tokens": 4, "enforce_eager": False},
                  {"ttft_ms": 16.0, "tpot_ms": 3.9, "e2e_ms": 500.0, "output_tokens_per_s": 24.0, "batch": 3, "stats": stats})
    # nine decode steps: three rounds of (all three decode, two left, one left); size 3 replays bucket 4, 2 bucket 2, 1 bucket 1
    rec["execution"] = {"backend": "cuda_graph", "graph_batch_sizes": [1, 2, 4], "decode_batch_sizes": {"3": 3, "2": 3, "1": 3},
                        "graph_replays": {"1": 3, "2": 3, "4": 3}, "eager_decode_steps": 0, "decode_steps": 9, "run_ahead": {"taken": 2, "discarded": 1}}
    rec["correctness"] = {"requests": 3, "output_tokens": 4, "output_token_ids": ids, "output_token_ids_sha256": canonical_json_sha256(ids),
                          "identical_across_repeats": True}
    rec["kv_cache"] = {"mode": "visual_compact_scaled_fp8", "kv_mode": 2, "page_tokens": 256, "pages": 64, "bytes_per_page": 1000,
                       "prompt_tokens": [300, 300, 520], "dropped_prompt_tokens": [60, 0, 10], "dense_prompt_bytes": 7000, "active_prompt_bytes": 5000}
    return rec


def test_system_record_carries_execution_correctness_and_kv_evidence():
    import copy

    good = _system_record()
    bs.validate_benchmark_record(good)
    for mutate, needle in (
        (lambda r: r["execution"]["graph_replays"].update({"4": 2}), "imply replays"),
        (lambda r: r["execution"].update(eager_decode_steps=1), "imply replays"),
        (lambda r: r["execution"]["decode_batch_sizes"].update({"8": 1}), "decode_steps is not the sum"),
        (lambda r: r["execution"]["graph_replays"].update({"3": 0}), "was not captured"),
        (lambda r: r["execution"].update(graph_batch_sizes=[4, 2, 1]), "ascending"),
        (lambda r: r["execution"].update(backend="eager"), "an eager run captured"),
        (lambda r: r["config"].update(enforce_eager=True), "contradicts"),
        (lambda r: r["correctness"]["output_token_ids"][0].pop(), "must hold 4"),
        (lambda r: r["correctness"]["output_token_ids"][1].__setitem__(0, 10), "sha256 does not match"),
        (lambda r: r["correctness"].update(identical_across_repeats=False), "different tokens"),
        (lambda r: r["correctness"].update(output_tokens=5), "must hold 5"),
        (lambda r: r["kv_cache"].update(dense_prompt_bytes=6000), "dense_prompt_bytes does not follow"),
        (lambda r: r["kv_cache"].update(active_prompt_bytes=7000), "active_prompt_bytes does not follow"),
        (lambda r: r["kv_cache"].update(mode="scaled_fp8_kv"), "does not compact"),
        (lambda r: r["kv_cache"]["dropped_prompt_tokens"].__setitem__(1, 300), "dropped 300 of 300"),
        (lambda r: r["results"]["stats"]["ttft_ms"].update(count=2), "3 rounds"),
        (lambda r: r["results"]["stats"]["tpot_ms"].update(p90=1.0), "does not hold"),
        (lambda r: r["results"].update(ttft_ms=15.0), "not the median"),
        (lambda r: r.pop("kv_cache"), "missing 'kv_cache'"),
    ):
        bad = copy.deepcopy(good)
        mutate(bad)
        with pytest.raises(bs.SchemaError, match=needle):
            bs.validate_benchmark_record(bad)
    # an eager run: every decode step eager, nothing captured; a batch beyond the largest bucket runs eagerly in graph mode
    eager = copy.deepcopy(good)
    eager["config"]["enforce_eager"] = True
    eager["execution"].update(backend="eager", graph_batch_sizes=[], graph_replays={}, eager_decode_steps=9)
    bs.validate_benchmark_record(eager)
    over = copy.deepcopy(good)
    over["execution"].update(graph_batch_sizes=[1, 2], decode_batch_sizes={"3": 3, "2": 3, "1": 3}, graph_replays={"1": 3, "2": 3}, eager_decode_steps=3)
    bs.validate_benchmark_record(over)


def test_mvbench_prompt_and_answer_extraction():
    from prism_infer_b200.analysis import quality_metrics as qm

    assert qm.mvbench_prompt("What does the person do?", ["runs", "jumps", "sits"]) == \
        "Question:What does the person do?\nOption:\n(A) runs\n(B) jumps\n(C) sits\nOnly give the best option.\n"
    with pytest.raises(ValueError):
        qm.mvbench_prompt("", ["a", "b"])
    with pytest.raises(ValueError):
        qm.mvbench_prompt("q", ["only one"])
    cases = {"B. the man walks": ("B", "leading_label_period"), "The answer is (C).": ("C", "embedded_label"), "a": ("A", "embedded_label"),
             "I think it's D, because 1,000 people": ("D", "embedded_label"), "none of them": (None, "unparseable"), "": (None, "unparseable"),
             "  d. because\nit moves": ("D", "embedded_label"), "[E]": ("E", "embedded_label")}
    for text, want in cases.items():
        assert qm.mvbench_choice(text) == want, text
    rec = {"candidates": ["runs", "jumps", "sits"], "answer_index": 1}
    hit, miss, silent = qm.mvbench_score(rec, "(B) jumps"), qm.mvbench_score(rec, "C"), qm.mvbench_score(rec, "  ")
    assert hit["score"] == 1 and hit["target"] == "B" and miss["score"] == 0 and not silent["answered"] and silent["prediction"] is None
    agg = qm.mvbench_accuracy([hit, miss, silent])
    assert agg == {"samples": 3, "accuracy": 1 / 3, "answered": 2 / 3, "unparseable": 1}
    assert qm.mvbench_accuracy([]) == {"samples": 0}
