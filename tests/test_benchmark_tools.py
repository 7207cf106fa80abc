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
            "model": "random:tiny", "data": "synthetic", "hardware": {"gpus": 1},
            "config": {"variant": "compact_prefix", "groups": 42, "questions": 85, "requests": 600, "rate_per_s": 4.0, "pages": 220,
                       "page_tokens": 256, "kv_budget_bytes": 220 * 1000, "working_set_pages": 148, "max_tokens": 16, "tp": 1},
            "results": {"ttft_p50_ms": ttft, "ttft_p99_ms": ttft * 2, "e2e_p50_ms": 80.0, "e2e_p99_ms": 120.0,
                        "recomputed_prompt_tokens": 100, "prompt_tokens": 5000, "output_tokens_per_s": 64.0, "completed": 600,
                        "duration_s": 150.0, "resident_media": 42, "prefix_evictions": 0, "prefix_hits": 500, "resident_pages": 148}}


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


def test_working_set_quality_runner_stages_resume_and_pairing(tmp_path):
    """Two media groups with two / three questions on the tiny model: both stages run, the
    repeat questions hit the stored prefix, an interrupted stage file resumes at a group
    boundary, a foreign file is refused."""
    import io

    import numpy as np
    import pytest
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import working_set_quality as wsq
    from prism_infer_b200.analysis.quality_materialization import materialize_image
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    q = _load("bench_working_set_quality")
    root = tmp_path / "media"
    rng = np.random.default_rng(0)

    def png(size):
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, (size, size, 3), dtype=np.uint8)).save(buf, format="PNG")
        return materialize_image(buf.getvalue(), root=root, dataset_id="synthetic")

    a, b, c = png(64), png(64), png(96)
    records = [
        {"sample_id": "s1", "question": "which is brighter", "options": ["left", "right"], "answer": "A", "media": [a, b]},
        {"sample_id": "s2", "question": "compare <image> with <image>", "options": ["same", "other", "none"], "answer": "C", "media": [a, b]},
        {"sample_id": "s3", "question": "read the sign", "answers": ["stop", "STOP sign"], "media": [c]},
        {"sample_id": "s4", "question": "what colour", "answers": ["red"], "media": [c]},
        {"sample_id": "s5", "question": "how many", "answers": ["one"], "media": [c]},
        {"sample_id": "lonely", "question": "alone", "answers": ["x"], "media": [b]},
    ]
    rec_path = tmp_path / "records.jsonl"
    rec_path.write_text("".join(json.dumps(r) + "\n" for r in records))
    loaded = q.load_records(rec_path)
    plan = wsq.select_multi_question_groups(loaded)
    assert len(plan) == 5 and {it.record["sample_id"] for it in plan} == {"s1", "s2", "s3", "s4", "s5"}
    assert q.prompt_for(loaded[1]).count("<image>") == 2 and "compare Image 1 with Image 2" in q.prompt_for(loaded[1])
    assert q.score(loaded[0], "The answer is (A).")["correct"] and not q.score(loaded[0], "B")["correct"]
    assert q.score(loaded[2], "Stop")["score"] == 1.0 and q.score(loaded[2], "yield")["score"] == 0.0
    with pytest.raises(ValueError):
        rec_bad = tmp_path / "bad.jsonl"
        rec_bad.write_text(json.dumps({"sample_id": 1, "question": "q", "media": [a]}) + "\n")
        q.load_records(rec_bad)

    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    built = []

    def make_engine(extra):
        extra = dict(extra)
        if "visual_pruning_min_keep_tokens" in extra:
            extra.update(visual_pruning_min_keep_tokens=2, visual_pruning_keep_ratio=0.5)
        built.append(extra["compression_mode"])
        return LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=128,
                   enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=True, **extra)

    out = tmp_path / "run"
    out.mkdir()
    quiet = lambda _m: None  # noqa: E731
    dense = q.run_stage("dense_prefix", plan, make_engine, root, out, max_tokens=3, resume=False, log=quiet)
    assert [r["sample_id"] for r in dense] == [it.record["sample_id"] for it in plan]
    assert [r["prefix_hit"] for r in dense] == [it.question_index > 0 for it in plan]
    assert all(r["deleted_visual_tokens"] == 0 for r in dense) and all(r["cached_tokens"] > 0 for r in dense if r["prefix_hit"])
    with pytest.raises(FileExistsError):
        q.run_stage("dense_prefix", plan, make_engine, root, out, max_tokens=3, resume=False, log=quiet)
    # an interrupted compact stage: the first group and one line of the second survive on disk
    compact_full = q.run_stage("compact_prefix", plan, make_engine, root, out, max_tokens=3, resume=False, log=quiet)
    assert any(r["deleted_visual_tokens"] > 0 for r in compact_full)
    first_group = plan[0].group_size
    path = out / "compact_prefix.samples.jsonl"
    path.write_text("".join(json.dumps(r) + "\n" for r in compact_full[:first_group + 1]))
    n_built = len(built)
    resumed = q.run_stage("compact_prefix", plan, make_engine, root, out, max_tokens=3, resume=True, log=quiet)
    assert resumed == compact_full and len(built) == n_built + 1
    assert q.run_stage("compact_prefix", plan, make_engine, root, out, max_tokens=3, resume=True, log=quiet) == compact_full
    assert len(built) == n_built + 1  # complete: no engine
    path.write_text(json.dumps(dict(compact_full[0], sample_id="zzz")) + "\n")
    with pytest.raises(ValueError, match="does not match the plan"):
        q.run_stage("compact_prefix", plan, make_engine, root, out, max_tokens=3, resume=True, log=quiet)
    summary = q.summarize({"dense_prefix": dense, "compact_prefix": compact_full}, plan)
    assert summary["samples"] == 5 and summary["groups"] == 2
    assert summary["stages"]["dense_prefix"]["repeat_prefix_hits"] == 3 == summary["stages"]["dense_prefix"]["repeat_questions"]
    assert summary["paired_deleted_subset"]["cohort"] == summary["stages"]["compact_prefix"]["samples_with_deletions"] > 0


def test_system_benchmark_cell_produces_a_record_that_satisfies_its_contract():
    """``bench_system.run_cell`` on the tiny model (CPU, eager): three rounds of two image requests, one dense and one
    compacting mode; the record carries the round statistics, eager-path evidence, repeatable token ids and the KV
    accounting of the prompts (dropped visual tokens only in the compacting mode)."""
    import numpy as np
    import torch

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import benchmark_schema as bs
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    b = _load("bench_system")
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    wl = {"name": "t", "kind": "image", "images": 1, "image_size": 224, "frames": 0, "question_tokens": 6, "output_tokens": 4}
    for mode, dropped_expected in (("eager_scaled_fp8_kv", False), ("eager_visual_compact", True)):
        opts = dict(enforce_eager=True, compression_mode="scaled_fp8_kv") if not dropped_expected else \
            dict(enforce_eager=True, compression_mode="visual_compact", visual_pruning_keep_ratio=0.5, visual_pruning_min_keep_tokens=2)
        llm = LLM("random:tiny", weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=64,
                  max_num_seqs=2, max_num_batched_tokens=256, max_chunk_size=256, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, **opts)
        cell = b.run_cell(llm, wl, 2, np.random.default_rng(0), repeats=3)
        llm.exit()
        rec = {"schema_version": bs.BENCHMARK_SCHEMA_VERSION, "benchmark": "system_mode_matrix", "engine": "prism_infer_b200", "model": "random:tiny",
               "data": "synthetic", "hardware": {"gpus": 1},
               "config": {"mode": mode, "workload": "t", "tp": 1, "repeats": 3, "output_tokens": 4, **opts},
               "results": cell["results"], "execution": cell["execution"], "correctness": cell["correctness"], "kv_cache": cell["kv_cache"]}
        bs.validate_benchmark_record(rec)
        ex = cell["execution"]
        assert ex["backend"] == "eager" and ex["decode_steps"] == ex["eager_decode_steps"] == 3 * 3 and ex["decode_batch_sizes"] == {"2": 9}
        assert cell["correctness"]["identical_across_repeats"] and len(cell["correctness"]["output_token_ids"]) == 2
        assert cell["results"]["stats"]["e2e_ms"]["count"] == 3
        assert any(cell["kv_cache"]["dropped_prompt_tokens"]) == dropped_expected
        assert (cell["kv_cache"]["active_prompt_bytes"] < cell["kv_cache"]["dense_prompt_bytes"]) == dropped_expected


def test_working_set_plan_from_materialised_records(tmp_path):
    """Real media groups: records over the same ordered files form a group, the page measurement reads the files
    (re-hashed), the plan document names them and the loader refuses a damaged file."""
    import io

    import numpy as np
    import pytest
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import working_set_plan as wsp
    from prism_infer_b200.analysis.identity import canonical_json_sha256
    from prism_infer_b200.analysis.quality_materialization import materialize_image
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    b = _load("build_working_set_plan")
    root = tmp_path / "media"
    rng = np.random.default_rng(3)

    def png(size):
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 256, (size, size, 3), dtype=np.uint8)).save(buf, format="PNG")
        return materialize_image(buf.getvalue(), root=root, dataset_id="synthetic")

    a, c, d = png(64), png(64), png(96)
    records = [
        {"sample_id": "s1", "question": "which is brighter", "options": ["left", "right"], "answer": "A", "media": [a, c]},
        {"sample_id": "s2", "question": "compare <image> with <image>", "options": ["same", "other"], "answer": "B", "media": [a, c]},
        {"sample_id": "s3", "question": "read the sign", "answers": ["stop"], "media": [d]},
        {"sample_id": "s4", "question": "what colour", "answers": ["red"], "media": [d]},
        {"sample_id": "s5", "question": "order matters", "answers": ["x"], "media": [c, a]},
    ]
    groups, paths = wsp.groups_from_records(records)
    assert len(groups) == 2 and sorted(g.num_images for g in groups) == [1, 2] and set(paths) == {a["sha256"], c["sha256"], d["sha256"]}
    two = next(g for g in groups if g.num_images == 2)
    assert two.questions[1].startswith("compare Image 1 with Image 2\n(A) same\n(B) other\n") and two.questions[1].endswith(wsp.CHOICE_HINT)
    assert two.group_id == wsp.group_id_of([a["sha256"], c["sha256"]])
    with pytest.raises(ValueError, match="duplicate sample id"):
        wsp.groups_from_records(records + [records[0]])

    contract = b.measurement_contract(model="random:tiny", page_tokens=16, image_size=0, seed=1, groups=groups,
                                      records_sha256=canonical_json_sha256(records))
    assert contract["media"] == "materialized_records"
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)

    def make_engine():
        return LLM("random:tiny", weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=128,
                   enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=True, compression_mode="scaled_fp8_kv")

    loader = b.file_image_loader(root, paths)
    art = b.measure_all(groups, tmp_path / "plan.json.pages.json", contract, make_engine, loader, resume=False, log=lambda _m: None)
    assert all(art["groups"][g.group_id]["dense_prefix_pages"] > 0 for g in groups)
    measured = [wsp.MediaGroup(g.group_id, g.media_digests, g.questions, art["groups"][g.group_id]["dense_prefix_pages"]) for g in groups]
    plan = wsp.build_plan(measured, num_requests=6, rate=50.0, seed=3, page_budget=4)
    doc = b.plan_document(plan, contract, "all", paths)
    assert set(doc["media_paths"]) == set(paths)
    (tmp_path / "plan.json").write_text(json.dumps(doc))
    loaded, doc2 = b.load_plan_document(tmp_path / "plan.json")
    assert doc2["media_paths"] == doc["media_paths"] and loaded.groups == plan.groups
    victim = root / paths[d["sha256"]]
    victim.write_bytes(victim.read_bytes() + b"0")
    with pytest.raises(OSError, match="mismatch"):
        loader(d["sha256"])


def test_online_benchmark_workload_options_and_profile(tmp_path):
    """``bench_online`` pieces on the tiny model: engine options from flags and key=value pairs, the three arrival
    processes, and a run with the SLO-aware policy, cooperative prefill, warm-up requests, deadlines and a profile file."""
    import argparse

    import torch

    from prism_infer_b200 import LLM
    from prism_infer_b200.analysis import online_serving
    from prism_infer_b200.analysis import working_set_plan as wsp
    from prism_infer_b200.analysis.performance_profile import validate_profile_record
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    b = _load("bench_online")
    ns = argparse.Namespace(variant="dense_prefix", engine_option=["max_num_seqs=4", "scheduler_policy=fcfs", "note=free text"],
                            **{flag.lstrip("-").replace("-", "_"): None for flag in b.ENGINE_FLAGS})
    ns.scheduler_policy, ns.enable_cooperative_prefill, ns.cooperative_prefill_coalesce_ms = "slo_aware", True, 0.0
    opts = b.engine_options(ns)
    assert opts["scheduler_policy"] == "fcfs" and opts["max_num_seqs"] == 4 and opts["note"] == "free text"  # key=value pairs win
    assert opts["enable_cooperative_prefill"] is True and opts["enable_prefix_caching"] is True and "cooperative_prefill_coalesce_ms" in opts
    groups = wsp.synthetic_groups(3, 7, seed=5, min_images=1, max_images=2, tokens_per_image=6, page=16)
    plan = wsp.build_plan(groups, num_requests=6, rate=200.0, seed=5, page_budget=64)
    assert b.arrival_offsets(plan, "burst", 200.0) == [0.0] * 6
    assert b.arrival_offsets(plan, "uniform", 200.0) == [i / 200.0 for i in range(6)]
    assert b.arrival_offsets(plan, "poisson", 200.0) == [r.arrival_offset_s for r in plan.measured]

    arch = Qwen3VLArch.tiny()
    llm = LLM("random:tiny", weights=random_weights(arch, dtype=torch.float32, seed=0), device="cpu", max_model_len=512, kvcache_block_size=16,
              num_kvcache_blocks=128, enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512, enable_prefix_caching=True,
              compression_mode="scaled_fp8_kv", scheduler_policy="slo_aware", enable_cooperative_prefill=True,
              cooperative_prefill_layer_quantum=1, max_num_seqs=4)
    prof = tmp_path / "profile.json"
    out = b.run_workload(llm, plan, lambda d: b.image_for(d, 64), max_tokens=3, arrival_process="uniform", rate=200.0, ttft_slo_ms=5000.0,
                         warmup_requests=2, profile_output=str(prof))
    summary = out["summary"]
    assert summary["requests"] == {"total": 6, "completed": 6, "rejected": 0, "cancelled": 0} and summary["output_tokens"] == 18
    assert summary["ttft_ms"]["count"] == 6 and summary["queue_ms"]["count"] in (0, 6)
    assert llm.multimodal_prefix_cache_metadata()["hits"] >= 6  # every measured request reuses its group's prefix
    validate_profile_record(json.loads(prof.read_text()))
    assert online_serving.summarize_online_run({"duration_s": out["result"].duration_s,
                                                "requests": [r.to_record() for r in out["result"].requests]})["requests_per_s"] > 0
    llm.exit()


def test_paged_decode_benchmark_sweeps_and_gates(tmp_path):
    """The paged-decode micro-benchmark on CPU: a sweep over cache formats, page size, context lengths and batch sizes
    writes one row per case with its difference to the plain-PyTorch statement; gates that cannot be met fail the run;
    an existing output is not overwritten silently."""
    import pytest

    b = _load("bench_paged_decode")
    out = tmp_path / "pd.json"
    common = ["--device", "cpu", "--batch-sizes", "1,3", "--context-lens", "37,64", "--page-sizes", "16", "--cache-dtypes", "scaled_fp8,fp8,bf16",
              "--num-heads", "4", "--num-kv-heads", "2", "--head-dim", "64", "--repeat", "1", "--warmup", "0"]
    assert b.main(common + ["--output", str(out)]) == 0
    rec = json.loads(out.read_text())
    assert rec["passed"] and len(rec["rows"]) == 3 * 2 * 2 and {r["cache_dtype"] for r in rec["rows"]} == {"scaled_fp8", "fp8", "bf16"}
    row = next(r for r in rec["rows"] if r["cache_dtype"] == "scaled_fp8" and r["batch"] == 3 and r["context_len"] == 37)
    assert row["kv_bytes"] == 2 * 3 * 37 * 2 * 64 * 1 + 2 * 3 * 37 * 2 * 4 and row["max_abs_diff"] <= 2e-2
    with pytest.raises(SystemExit):
        b.main(common + ["--output", str(out)])                       # exists
    assert b.main(common + ["--output", str(out), "--overwrite", "--max-abs-diff", "-1"]) == 1
    assert json.loads(out.read_text())["passed"] is False
    with pytest.raises(SystemExit):
        b.main(["--device", "cpu", "--cache-dtypes", "int4"])


def test_kv_capacity_accounting_and_measured_mode(tmp_path, capsys):
    """Accounting gives the documented ratio; the measured mode on the tiny model shows the scaled-FP8 engine holding about
    twice the sequences of the bf16 engine at the same byte budget."""
    b = _load("bench_kv_capacity")
    acc = b.accounting("random:qwen3-vl-8b", 4_282_122_240, 1)
    assert acc["off"]["pages"] == 113 and acc["scaled_fp8_kv"]["pages"] == 220 and acc["scaled_over_bf16_bytes"] == 0.515625
    manifest = {"schema_version": 1, "name": "t", "cases": [{"id": "img", "requests": [
        {"type": "image", "prompt": "7 8 9", "image": {"width": 224, "height": 224, "seed": 1}}]}]}
    path = tmp_path / "m.json"
    path.write_text(json.dumps(manifest))
    tiny_acc = b.accounting("random:tiny", 10 * 1024 * 1024, 1, page_tokens=16, modes=("off", "scaled_fp8_kv"))
    rc = b.main(["--measure", "--model", "random:tiny", "--device", "cpu", "--budget-bytes", str(24 * tiny_acc["off"]["bytes_per_page"]),
                 "--page-tokens", "16", "--manifest", str(path), "--case", "img", "--requests", "6", "--max-tokens", "3", "--max-model-len", "256",
                 "--modes", "off", "scaled_fp8_kv", "--output", str(tmp_path / "cap.json")])
    capsys.readouterr()
    assert rc == 0
    rec = json.loads((tmp_path / "cap.json").read_text())
    dense, scaled = rec["measured"]
    assert dense["pages"] == 24 and scaled["pages"] == int(24 / 0.53125) == 45  # 64-wide heads: one fp32 scale per 64 payload bytes
    assert dense["completed"] == scaled["completed"] == 6 and dense["prompt_pages_per_request"] == scaled["prompt_pages_per_request"] == 4
    assert dense["sequences_that_fit_by_pages"] == 6 and scaled["sequences_that_fit_by_pages"] == 11
    assert scaled["preempted"] == 0 and scaled["peak_resident_sequences"] == 6


def test_system_benchmark_main_sweeps_on_the_tiny_model(tmp_path, capsys):
    """``bench_system.main`` end to end on CPU: two eager modes (one of them dropping visual tokens at two keep ratios),
    two batch sizes and two output lengths on the text workload give one valid record per cell, and the profile of the
    last cell is written."""
    from prism_infer_b200.analysis import benchmark_schema as bs
    from prism_infer_b200.analysis.performance_profile import validate_profile_record

    b = _load("bench_system")
    out, prof = tmp_path / "records.json", tmp_path / "profile.json"
    b.main(["--model", "random:tiny", "--device", "cpu", "--modes", "eager", "eager_visual_prune", "--workloads", "text_256", "--batch-sizes", "1", "2",
            "--output-lengths", "2", "3", "--visual-pruning-keep-ratios", "0.5", "0.75", "--repeats", "2", "--page-tokens", "16",
            "--max-model-len", "512", "--out", str(out), "--profile-output", str(prof), "--quiet"])
    assert capsys.readouterr().out == ""
    records = json.loads(out.read_text())
    assert len(records) == (1 + 2) * 2 * 2  # the pruning mode once per keep ratio
    for rec in records:
        bs.validate_benchmark_record(rec)
    assert {(r["config"]["mode"], r["config"].get("visual_pruning_keep_ratio")) for r in records} == \
        {("eager", None), ("eager_visual_prune", 0.5), ("eager_visual_prune", 0.75)}
    assert {r["results"]["batch"] for r in records} == {1, 2} and {r["config"]["output_tokens"] for r in records} == {2, 3}
    validate_profile_record(json.loads(prof.read_text()))


def test_external_engine_arm_builds_requests_and_times_a_fake_engine(capsys):
    """The vLLM arm's adapter with a fake engine: media-first token-id prompts with one placeholder per image, fresh
    inputs for every timed call, TPOT from the difference of two runs, a refusal when the engine ignores ``ignore_eos``;
    and, on a box without a CUDA device, the ``unavailable`` line instead of a crash."""
    import numpy as np
    import pytest
    import torch

    from prism_infer_b200.models.architecture import Qwen3VLArch

    b = _load("bench_external_vllm")
    arch = Qwen3VLArch.qwen3_vl_8b()
    reqs = b.make_requests(arch, np.random.default_rng(0), batch=2, images=3, size=32, question_tokens=5)
    ids = reqs[0]["prompt_token_ids"]
    assert ids[:9] == [arch.vision_start_token_id, arch.image_token_id, arch.vision_end_token_id] * 3 and len(ids) == 9 + 5
    assert len(reqs[0]["multi_modal_data"]["image"]) == 3 and reqs[0]["multi_modal_data"]["image"][0].size == (32, 32)
    assert "multi_modal_data" not in b.make_requests(arch, np.random.default_rng(0), batch=1, images=0, size=32, question_tokens=4)[0]
    now, calls, made = [0.0], [], []

    def make():
        made.append(len(made))
        return [{"prompt_token_ids": [made[-1]]}]

    def generate(prompts, max_tokens):  # 10 ms prefill + 2 ms per token after the first
        calls.append((prompts[0]["prompt_token_ids"][0], max_tokens))
        now[0] += 0.010 + 0.002 * (max_tokens - 1)
        return [[7] * max_tokens for _ in prompts]

    res = b.measure(generate, make, output_tokens=20, warmup=1, repeats=3, clock=lambda: now[0])
    assert abs(res["ttft_ms"] - 10.0) < 1e-6 and abs(res["tpot_ms"] - 2.0) < 1e-6 and abs(res["e2e_ms"] - 50.0) < 1e-6
    assert [c[1] for c in calls] == [2, 1, 21, 1, 21, 1, 21] and len({c[0] for c in calls}) == 7  # never the same inputs twice
    with pytest.raises(RuntimeError, match="ignore_eos"):
        b.measure(lambda p, n: [[1] * min(n, 5) for _ in p], make, output_tokens=20, warmup=0, repeats=1)
    if not torch.cuda.is_available():
        assert b.main([]) == 0
        line = json.loads(capsys.readouterr().out)
        assert line == {"engine": "vllm", "unavailable": "no CUDA device"}


def test_decode_matrix_and_ttft_benchmarks_run_end_to_end_on_cpu(tmp_path, capsys):
    """The two latency benchmarks through their command-line entries on the tiny model: the decode matrix writes a record
    that satisfies its contract; the TTFT breakdown prints the engine's profile regions per request for images and for a
    chunked long text prompt."""
    from prism_infer_b200.analysis import benchmark_schema as bs

    d = _load("bench_decode")
    out = tmp_path / "decode.json"
    d.main(["--model", "random:tiny", "--device", "cpu", "--workload", "image1", "--image-size", "64", "--batches", "1,2", "--output-tokens", "12",
            "--out", str(out)])
    rec = json.loads(out.read_text())
    bs.validate_benchmark_record(rec)
    assert [r["batch"] for r in rec["results"]["rows"]] == [1, 2] and "steady_step_ms_median" in rec["results"]["rows"][1]
    capsys.readouterr()
    t = _load("bench_ttft")
    t.main(["--model", "random:tiny", "--device", "cpu", "--images", "2", "--image-size", "64", "--repeats", "2"])
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["workload"] == "images2" and len(line["ttft_ms"]) == 2 and line["regions"]["engine.step"]["count_per_request"] >= 1
    t.main(["--model", "random:tiny", "--device", "cpu", "--text-tokens", "300", "--chunk", "128", "--repeats", "2", "--paged-prefill-kernel", "both"])
    lines = [json.loads(x) for x in capsys.readouterr().out.strip().splitlines()]
    assert [x["workload"] for x in lines] == ["text300_chunk128_tc", "text300_chunk128_mma"] and all(x["prompt_tokens"] == 300 for x in lines)
