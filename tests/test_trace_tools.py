"""Nsight Systems export reader on a fabricated SQLite file, and the cold -> prefix-hit trace
with its evidence and audit on the tiny model (CPU)."""

import importlib.util
import json
import os
import sqlite3

import numpy as np
import pytest
import torch

from prism_infer_b200.analysis import nsys_trace, prefix_trace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "benchmarks", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _fabricate_export(path, *, hit_has_vision=False):
    """Two engine steps (one prefill with plain launches, one decode as a graph replay), marker
    ranges for a cold and a prefix-hit request, strings partly inline and partly by id."""
    con = sqlite3.connect(path)
    con.executescript("""
        CREATE TABLE StringIds (id INTEGER PRIMARY KEY, value TEXT);
        CREATE TABLE NVTX_EVENTS (start INTEGER, end INTEGER, text TEXT, textId INTEGER, eventType INTEGER);
        CREATE TABLE CUPTI_ACTIVITY_KIND_RUNTIME (start INTEGER, end INTEGER, correlationId INTEGER, nameId INTEGER);
        CREATE TABLE CUPTI_ACTIVITY_KIND_KERNEL (start INTEGER, end INTEGER, correlationId INTEGER, shortName INTEGER, demangledName INTEGER);
        CREATE TABLE CUPTI_ACTIVITY_KIND_MEMCPY (start INTEGER, end INTEGER, correlationId INTEGER, bytes INTEGER);
        CREATE TABLE CUPTI_ACTIVITY_KIND_GRAPH_TRACE (start INTEGER, end INTEGER, correlationId INTEGER, graphId INTEGER);
    """)
    strings = {1: "cudaLaunchKernelExC_v11060", 2: "cudaGraphLaunch_v10000", 3: "cudaMemcpyAsync_v3020", 4: "cudaStreamSynchronize_v3020",
               10: "gemm_wx_persistent_kernel<256, false, true>", 11: "flash_tc_kernel<128>", 12: "sample_kernel", 13: "mystery",
               20: "prism::engine.step", 21: "prism::model.vision.encoder"}
    con.executemany("INSERT INTO StringIds VALUES (?, ?)", strings.items())
    nvtx = [
        (1000, 99000, "prism::cold_request", None), (100000, 160000, "prism::prefix_hit_request", None),
        (2000, 50000, None, 20),       # prefill step (by string id)
        (3000, 9000, None, 21),        # vision range inside the cold request
        (60000, 70000, "prism::engine.step", None),   # decode step (inline text)
        (110000, 150000, "prism::engine.step", None),  # the hit's prefill step
        (5000, None, "open range", None),
    ]
    if hit_has_vision:
        nvtx.append((111000, 112000, "prism::model.vision.encoder", None))
    con.executemany("INSERT INTO NVTX_EVENTS VALUES (?, ?, ?, ?, 59)", [(s, e, t, i) for s, e, t, i in nvtx])
    runtime = [  # start, end, correlation, name id
        (2500, 2600, 1, 3), (4000, 4100, 2, 1), (4200, 4300, 3, 1), (4400, 4500, 4, 1), (49000, 49500, 5, 4),
        (61000, 61200, 6, 2), (120000, 120100, 7, 1),
    ]
    con.executemany("INSERT INTO CUPTI_ACTIVITY_KIND_RUNTIME VALUES (?, ?, ?, ?)", runtime)
    kernels = [(5000, 15000, 2, 10, 10), (14000, 30000, 3, 11, 11), (52000, 53000, 4, 12, 12), (121000, 126000, 7, 13, 13)]
    con.executemany("INSERT INTO CUPTI_ACTIVITY_KIND_KERNEL VALUES (?, ?, ?, ?, ?)", kernels)
    con.execute("INSERT INTO CUPTI_ACTIVITY_KIND_MEMCPY VALUES (2700, 3700, 1, 4096)")
    con.execute("INSERT INTO CUPTI_ACTIVITY_KIND_GRAPH_TRACE VALUES (62000, 66000, 6, 1)")
    con.commit()
    con.close()


def test_nsys_export_summary(tmp_path):
    path = str(tmp_path / "capture.sqlite")
    _fabricate_export(path)
    out = nsys_trace.analyze_nsys_sqlite(path, prefill_steps=1, target_ranges=["prism::model.vision.encoder", "prism::absent"])
    assert out["record_type"] == "nsys_profile_summary" and len(out["raw_steps"]) == 3
    pre = out["raw_steps"][0]
    assert pre["kernel_count"] == 3 and pre["kernel_launch_api_count"] == 3 and pre["memcpy_async_count"] == 1
    assert pre["stream_synchronize_count"] == 1 and pre["memcpy_bytes"] == 4096
    assert pre["kernel_time_ms"] == pytest.approx((10000 + 16000 + 1000) / 1e6)
    # busy time is the union: copy 1 us, kernels 5-30 us overlapping by 1 us, sampler 1 us
    assert pre["gpu_busy_ms"] == pytest.approx((1000 + 25000 + 1000) / 1e6)
    assert pre["gpu_tail_after_cpu_ms"] == pytest.approx(3000 / 1e6)   # the sampler ran after the CPU range closed
    assert pre["launch_to_kernel_median_us"] == pytest.approx(9.7)      # gaps 0.9, 9.7, 47.5 us
    assert pre["kernel_categories"]["gemm_tcgen05"]["count"] == 1 and pre["kernel_categories"]["attention_prefill"]["count"] == 1
    dec = out["raw_steps"][1]
    assert dec["graph_launch_api_count"] == 1 and dec["graph_execution_ms"] == pytest.approx(0.004) and dec["kernel_count"] == 0
    assert out["phase_summary"]["prefill"]["steps"] == 1 and out["phase_summary"]["decode"]["steps"] == 2
    assert out["target_ranges"]["prism::model.vision.encoder"]["occurrences"] == 1
    assert out["target_ranges"]["prism::model.vision.encoder"]["kernel_count"]["total"] == 3
    assert out["target_ranges"]["prism::absent"] == {"occurrences": 0}
    assert out["top_kernels"][0]["name"].startswith("flash_tc_kernel") and [k["category"] for k in out["top_kernels"]] == [
        "attention_prefill", "gemm_tcgen05", "other", "sampler"]
    with pytest.raises(ValueError):
        nsys_trace.analyze_nsys_sqlite(path, prefill_steps=3)
    empty = str(tmp_path / "empty.sqlite")
    sqlite3.connect(empty).execute("CREATE TABLE StringIds (id INTEGER, value TEXT)").connection.commit()
    with pytest.raises(ValueError, match="missing tables"):
        nsys_trace.analyze_nsys_sqlite(empty)
    assert nsys_trace.union_ns([(0, 10), (5, 20), (30, 40), (40, 35)]) == 30
    assert nsys_trace.percentile([1, 2, 3, 4], 0.5) == 2.5
    assert nsys_trace.kernel_category("void prism::add_rmsnorm_rows_kernel<8>") == "norm_rope_kv"


def test_analyze_nsys_cli_refuses_to_overwrite(tmp_path, monkeypatch, capsys):
    path = str(tmp_path / "capture.sqlite")
    _fabricate_export(path)
    cli = _load("analyze_nsys")
    out = str(tmp_path / "summary.json")
    monkeypatch.setattr("sys.argv", ["analyze_nsys.py", path, "--output", out, "--quiet"])
    cli.main()
    assert json.load(open(out))["prefill_steps"] == 1 and capsys.readouterr().out == ""
    with pytest.raises(FileExistsError):
        cli.main()


def _evidence_inputs():
    zero = {k: 0 for k in prefix_trace.PREFIX_COUNTERS}
    after_cold = dict(zero, probes=1, misses=1, stores=1)
    after_hit = dict(after_cold, probes=2, probe_hits=1, hits=1)
    cold = {"finish_reason": "length", "cached_tokens": 0, "prompt_tokens": 60}
    hit = {"finish_reason": "length", "cached_tokens": 50, "prompt_tokens": 61}
    return zero, after_cold, after_hit, cold, hit


def test_prefix_hit_evidence_fails_closed():
    zero, after_cold, after_hit, cold, hit = _evidence_inputs()
    ok = prefix_trace.validate_prefix_hit_evidence(zero, after_cold, after_hit, cold, hit, cold_vision_patches=196, hit_vision_patches=0)
    assert ok["passed"] and ok["cached_fraction"] == pytest.approx(50 / 61)
    bad_cases = [
        dict(after_cold=dict(after_cold, hits=1)),                       # the cold request hit
        dict(after_cold=dict(after_cold, stores=0)),                     # nothing stored
        dict(after_hit=dict(after_hit, probe_hits=0)),                   # no probe hit
        dict(after_hit=dict(after_hit, misses=2)),                       # hit request missed
        dict(after_hit=dict(after_hit, stale_probes=1)),                 # stale fallback
        dict(after_hit=dict(after_hit, probes=0)),                       # a counter went backwards
        dict(hit=dict(hit, cached_tokens=0)), dict(hit=dict(hit, cached_tokens=99)), dict(hit=dict(hit, finish_reason="cancelled")),
        dict(cold=dict(cold, cached_tokens=4)), dict(hit_vision_patches=16), dict(cold_vision_patches=0),
    ]
    for change in bad_cases:
        args = dict(before=zero, after_cold=after_cold, after_hit=after_hit, cold=cold, hit=hit, cold_vision_patches=196, hit_vision_patches=0)
        args.update(change)
        with pytest.raises(ValueError):
            prefix_trace.validate_prefix_hit_evidence(args["before"], args["after_cold"], args["after_hit"], args["cold"], args["hit"],
                                                      cold_vision_patches=args["cold_vision_patches"], hit_vision_patches=args["hit_vision_patches"])


def test_audit_of_nsys_export_markers(tmp_path):
    zero, after_cold, after_hit, cold, hit = _evidence_inputs()
    evidence = prefix_trace.validate_prefix_hit_evidence(zero, after_cold, after_hit, cold, hit, cold_vision_patches=196, hit_vision_patches=0)
    tool = _load("trace_prefix_hit")
    good = str(tmp_path / "good.sqlite")
    _fabricate_export(good)
    audit = tool.audit_nsys_export(good, {"evidence": evidence})
    assert audit["passed"] and audit["cold_vision_ranges"] == {"model.vision.encoder": 1}
    assert audit["prefix_hit_nested_ranges"] == {"engine.step": 1}
    bad = str(tmp_path / "bad.sqlite")
    _fabricate_export(bad, hit_has_vision=True)
    with pytest.raises(RuntimeError, match="prefix_hit_trace_contains_no_vision"):
        tool.audit_nsys_export(bad, {"evidence": evidence})


def test_cold_then_prefix_hit_trace_on_tiny_model():
    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    tool = _load("trace_prefix_hit")
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    rng = np.random.default_rng(1)
    img = lambda: [rng.integers(0, 256, (64, 64, 3), dtype=np.uint8) for _ in range(2)]  # noqa: E731
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    llm = LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
              enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512)
    try:
        rec = tool.run_prefix_trace(llm, img(), img(), [5, 6, 7], [8, 9, 10, 11], sp)
        assert rec["audit"]["passed"] and rec["evidence"]["actual_cached_tokens"] > 0
        assert rec["evidence"]["prefix_hit_request_vision_patches"] == 0 and rec["evidence"]["cold_request_vision_patches"] == 32
        assert "model.vision.encoder" in rec["audit"]["cold_vision_ranges"] and not rec["audit"]["prefix_hit_vision_ranges"]
        assert rec["prefix_hit_request"]["first_token_wall_ms"] > 0
        with pytest.raises(ValueError, match="different questions"):
            tool.run_prefix_trace(llm, img(), img(), [1, 2], [1, 2], sp)
    finally:
        llm.exit()
    # with prefix caching off the second request re-encodes: the evidence refuses it
    llm = LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
              enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=False)
    try:
        with pytest.raises(ValueError):
            tool.run_prefix_trace(llm, img(), img(), [5, 6, 7], [8, 9, 10, 11], sp)
    finally:
        llm.exit()
