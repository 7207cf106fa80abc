"""Repeated-visual-context online serving benchmark (the working-set study).

42 media groups of 1-8 synthetic 448x448 images, 85 random-token questions, media-first
prompts; one warm-up request per group builds its prefix; then a measured open-loop stream
(default 600 requests, groups by Zipf(1.0), a different question than the group's previous
request, Poisson arrivals at 4 req/s, 16 output tokens) runs against a fixed KV budget
(default 220 pages of 256 tokens of scaled-FP8 KV) with the compact-prefix cache.
Reports TTFT p50/p99, end-to-end p50/p99, recomputed prompt tokens and output tokens/s, in
the reference's definitions (``benchmarks/bench_online.py`` and
``analysis/working_set_plan.py`` there).

    python benchmarks/bench_online.py --variant compact_prefix [--requests 600] [--rate 4] [--tp 1] [--out rec.json]

Engine options are flags of their own (``--scheduler-policy slo_aware --ttft-slo-ms 500``, ``--enable-cooperative-prefill
--cooperative-prefill-layer-quantum 4 --cooperative-prefill-coalesce-ms 250``, batch and queue limits) or go through
``--engine-option key=value`` (repeatable; the value is read as JSON, else as a string).  ``--arrival-process`` replaces
the plan's Poisson arrivals by evenly spaced ones or one burst; ``--warmup-requests`` runs that many untimed requests
before the population phase; ``--profile-output`` writes the performance profile of the measured stream.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from prism_infer_b200 import LLM, SamplingParams  # noqa: E402
from prism_infer_b200.analysis import benchmark_schema, online_serving, working_set_plan as wsp  # noqa: E402
import harness  # noqa: E402
from prism_infer_b200.engine.online import OnlineRequest, OnlineServingSession  # noqa: E402

VARIANTS = {
    "vision_only": dict(enable_prefix_caching=False, compression_mode="scaled_fp8_kv", enable_visual_embedding_cache=True),
    "dense_prefix": dict(enable_prefix_caching=True, compression_mode="scaled_fp8_kv", enable_visual_embedding_cache=True),
    "compact_prefix": dict(enable_prefix_caching=True, compression_mode="visual_compact_scaled_fp8",
                           enable_visual_embedding_cache=True, visual_pruning_keep_ratio=0.6,
                           visual_pruning_min_keep_tokens=768),
}


def image_for(digest: str, size: int) -> np.ndarray:
    seed = int.from_bytes(hashlib.sha256(digest.encode()).digest()[:8], "little")
    return np.random.default_rng(seed).integers(0, 256, (size, size, 3), dtype=np.uint8)


ENGINE_FLAGS = {  # flag -> (LLM keyword, type); None: a store_true switch
    "--scheduler-policy": ("scheduler_policy", str), "--max-num-seqs": ("max_num_seqs", int),
    "--max-num-batched-tokens": ("max_num_batched_tokens", int), "--max-chunk-size": ("max_chunk_size", int),
    "--max-model-len": ("max_model_len", int), "--max-queue-size": ("max_queue_size", int),
    "--max-consecutive-prefill-batches": ("max_consecutive_prefill_batches", int),
    "--min-decode-batches-between-heavy-prefills": ("min_decode_batches_between_heavy_prefills", int),
    "--max-light-prefill-bypasses-per-heavy": ("max_light_prefill_bypasses_per_heavy", int),
    "--heavy-prefill-vision-patch-threshold": ("heavy_prefill_vision_patch_threshold", int),
    "--cooperative-prefill-layer-quantum": ("cooperative_prefill_layer_quantum", int),
    "--cooperative-prefill-vision-block-quantum": ("cooperative_prefill_vision_block_quantum", int),
    "--cooperative-prefill-coalesce-ms": ("cooperative_prefill_coalesce_ms", float),
    "--logits-precision": ("logits_precision", str), "--visual-pruning-keep-ratio": ("visual_pruning_keep_ratio", float),
    "--visual-pruning-min-keep-tokens": ("visual_pruning_min_keep_tokens", int),
    "--visual-pruning-strategy": ("visual_pruning_strategy", str), "--image-max-pixels": ("image_max_pixels", int),
    "--enable-cooperative-prefill": ("enable_cooperative_prefill", None),
    "--enable-vision-tensor-cudagraph": ("enable_vision_tensor_cudagraph", None),
}
ENGINE_DEFAULTS = dict(max_model_len=8192, max_num_batched_tokens=8192, max_num_seqs=8, max_chunk_size=8192, cpu_kv_cache_ratio=0.0)


def engine_options(args) -> dict:
    """Variant, then the defaults of this benchmark, then explicit flags, then ``--engine-option`` pairs (last wins)."""
    opts = {**ENGINE_DEFAULTS, **VARIANTS[args.variant]}
    for flag, (key, _kind) in ENGINE_FLAGS.items():
        value = getattr(args, flag.lstrip("-").replace("-", "_"))
        if value is not None and value is not False:  # 0 and 0.0 are values
            opts[key] = value
    for pair in args.engine_option or []:
        key, sep, raw = pair.partition("=")
        if not sep or not key:
            raise SystemExit(f"--engine-option takes key=value, got {pair!r}")
        try:
            opts[key] = json.loads(raw)
        except json.JSONDecodeError:
            opts[key] = raw
    return opts


def arrival_offsets(plan: wsp.WorkingSetPlan, process: str, rate: float) -> list[float]:
    """``poisson``: the plan's own draws; ``uniform``: one request every 1 / rate seconds; ``burst``: all at once."""
    n = len(plan.measured)
    if process == "poisson":
        return [r.arrival_offset_s for r in plan.measured]
    if process == "uniform":
        return [i / rate for i in range(n)]
    if process == "burst":
        return [0.0] * n
    raise ValueError(f"unknown arrival process {process!r}")


def run_workload(llm, plan: wsp.WorkingSetPlan, load_image, *, max_tokens: int, arrival_process: str = "poisson", rate: float = 4.0,
                 ttft_slo_ms: float | None = None, warmup_requests: int = 0, profile_output: str = "") -> dict:
    """Warm-up, population (closed loop, one request per group), then the measured open-loop stream.  Returns the run
    result, the summary and the times of the phases."""
    session = OnlineServingSession(llm)
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    images = {g.group_id: [load_image(d) for d in g.media_digests] for g in plan.groups}

    def payload(r: wsp.PlannedRequest, question: str | None = None) -> dict:
        g = plan.groups[r.group_index]
        return {"type": "interleaved_images", "prompt": wsp.media_first_prompt(g.num_images, question or g.questions[r.question_index]),
                "images": images[g.group_id], "image_marker": wsp.IMAGE_MARKER}

    try:
        for i in range(warmup_requests):  # untimed: lazy initialisation, graph capture of new shapes; a question of its own
            r = plan.population[i % len(plan.population)]
            session.run([OnlineRequest(f"warmup-{i:03d}", 0.0, payload(r, f"{11 + i} {12 + i} {13 + i}"), sp)])
        t0 = time.perf_counter()
        for r in plan.population:
            session.run([OnlineRequest(r.request_key, 0.0, payload(r), sp)])
        population_s = time.perf_counter() - t0
        session.reset_metrics()
        offsets = arrival_offsets(plan, arrival_process, rate)
        stream = [OnlineRequest(r.request_key, off, payload(r), sp, ttft_slo_ms=ttft_slo_ms) for r, off in zip(plan.measured, offsets)]
        if profile_output:
            from prism_infer_b200.analysis.performance_profile import performance_profile, validate_profile_record
            from prism_infer_b200.analysis.quality_materialization import write_json_atomic

            with performance_profile({"benchmark": "online_working_set", "requests": len(stream)}, nvtx=False) as prof:
                result = session.run(stream)
            write_json_atomic(profile_output, validate_profile_record(prof.finalize()))
        else:
            result = session.run(stream)
        summary = online_serving.summarize_online_run({
            "duration_s": result.duration_s, "requests": [r.to_record() for r in result.requests],
            "scheduler_metrics": llm.metrics_snapshot()["scheduler"]})
    finally:
        session.close()
    return {"result": result, "summary": summary, "population_s": population_s}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--variant", choices=sorted(VARIANTS), default="compact_prefix")
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--requests", type=int, default=600)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--alpha", type=float, default=1.0)
    ap.add_argument("--groups", type=int, default=42)
    ap.add_argument("--questions", type=int, default=85)
    ap.add_argument("--pages", type=int, default=220)
    ap.add_argument("--page-tokens", type=int, default=256)
    ap.add_argument("--min-images", type=int, default=1)
    ap.add_argument("--max-images", type=int, default=8)
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--seed", type=int, default=wsp.DEFAULT_SEED)
    ap.add_argument("--plan", default="", help="plan document from build_working_set_plan.py (measured prefix pages); "
                                               "its groups, budget, rate and seed replace the flags above")
    ap.add_argument("--out", default="")
    ap.add_argument("--media-root", default="", help="root of the materialised media tree, for a plan built from real records")
    ap.add_argument("--device", default=None)
    ap.add_argument("--arrival-process", choices=("poisson", "uniform", "burst"), default="poisson")
    ap.add_argument("--ttft-slo-ms", type=float, default=None, help="first-token deadline of every measured request (slo_aware policy)")
    ap.add_argument("--warmup-requests", type=int, default=0)
    ap.add_argument("--profile-output", default="")
    ap.add_argument("--engine-option", action="append", default=None, metavar="KEY=VALUE")
    for flag, (_key, kind) in ENGINE_FLAGS.items():
        if kind is None:
            ap.add_argument(flag, action="store_true")
        else:
            ap.add_argument(flag, type=kind, default=None)
    args = ap.parse_args()

    plan_sha256 = None
    load_image = None
    if args.plan:
        from build_working_set_plan import load_plan_document

        plan, doc = load_plan_document(args.plan)
        plan_sha256 = doc["plan_sha256"]
        args.image_size, args.seed = doc["contract"]["image_size"], plan.seed
        args.pages, args.rate, args.alpha = plan.page_budget, plan.rate, plan.alpha
        args.groups, args.questions = doc["groups"], doc["questions"]
        args.requests = len(plan.measured)
        if "media_paths" in doc:  # real media: read (and re-hash) the files the plan names
            if not args.media_root:
                ap.error("this plan was built from materialised records: pass --media-root")
            from build_working_set_plan import file_image_loader

            load_image = file_image_loader(args.media_root, doc["media_paths"])
    else:
        groups = wsp.synthetic_groups(args.groups, args.questions, seed=args.seed, min_images=args.min_images,
                                      max_images=args.max_images, tokens_per_image=(args.image_size // 32) ** 2 + 2)
        plan = wsp.build_plan(groups, num_requests=args.requests, alpha=args.alpha, rate=args.rate, seed=args.seed,
                              page_budget=args.pages)
    options = engine_options(args)
    llm = LLM(args.model, device=args.device, tensor_parallel_size=args.tp, kvcache_block_size=args.page_tokens,
              num_kvcache_blocks=args.pages, **options)
    if not llm.is_driver:
        llm.serve_forever()
        return
    load_image = load_image or (lambda d: image_for(d, args.image_size))
    out = run_workload(llm, plan, load_image, max_tokens=args.max_tokens, arrival_process=args.arrival_process, rate=args.rate,
                       ttft_slo_ms=args.ttft_slo_ms, warmup_requests=args.warmup_requests, profile_output=args.profile_output)
    result, summary = out["result"], out["summary"]
    prefix = llm.multimodal_prefix_cache_metadata()
    record = {
        "schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "online_working_set",
        "engine": "prism_infer_b200", "model": args.model, "data": "synthetic" if not args.media_root else "materialized records",
        "hardware": {"gpus": args.tp},
        "provenance": harness.provenance(),
        "config": {"variant": args.variant, "groups": args.groups, "questions": args.questions, "requests": args.requests,
                   "rate_per_s": args.rate, "alpha": args.alpha, "pages": args.pages, "page_tokens": args.page_tokens,
                   "images_per_group": [args.min_images, args.max_images],
                   "kv_budget_bytes": args.pages * llm.config.kv_bytes_per_page(), "working_set_pages": plan.working_set_pages,
                   "max_tokens": args.max_tokens, "seed": args.seed, "tp": args.tp, "plan_sha256": plan_sha256,
                   "arrival_process": args.arrival_process, "ttft_slo_ms": args.ttft_slo_ms, "warmup_requests": args.warmup_requests,
                   "engine_options": {k: v for k, v in sorted(options.items())}},
        "results": {
            "ttft_p50_ms": summary["ttft_ms"]["p50"], "ttft_p99_ms": summary["ttft_ms"]["p99"],
            "e2e_p50_ms": summary["e2e_ms"]["p50"], "e2e_p99_ms": summary["e2e_ms"]["p99"],
            "recomputed_prompt_tokens": summary["recomputed_prompt_tokens"], "prompt_tokens": summary["prompt_tokens"],
            "output_tokens_per_s": summary["output_tokens_per_s"], "completed": summary["requests"]["completed"],
            "duration_s": result.duration_s, "population_s": out["population_s"],
            "resident_media": prefix["entries"], "prefix_evictions": prefix["evictions"], "prefix_hits": prefix["hits"],
            "resident_pages": prefix["resident_pages"], "media_cache": result.cache_counters,
            "cooperative_prefill": llm.cooperative_prefill_policy_metadata(),
        },
    }
    if args.ttft_slo_ms is not None:
        ttfts = [r.ttft_ms for r in result.requests if r.ttft_ms is not None]
        record["results"]["ttft_slo_attainment"] = sum(t <= args.ttft_slo_ms for t in ttfts) / max(1, len(ttfts))
    benchmark_schema.validate_benchmark_record(record)
    print(json.dumps(record["results"]), flush=True)
    if args.out:
        benchmark_schema.write_record(args.out, record)
    llm.exit()


if __name__ == "__main__":
    main()
