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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--variant", choices=sorted(VARIANTS), default="compact_prefix")
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--requests", type=int, default=600)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--alpha", type=float, default=1.0)
    ap.add_argument("--groups", type=int, default=42)
    ap.add_argument("--questions", type=int, default=85)
    ap.add_argument("--pages", type=int, default=220)
    ap.add_argument("--min-images", type=int, default=1)
    ap.add_argument("--max-images", type=int, default=8)
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--seed", type=int, default=wsp.DEFAULT_SEED)
    ap.add_argument("--plan", default="", help="plan document from build_working_set_plan.py (measured prefix pages); "
                                               "overrides the group, request, rate, seed and page arguments")
    ap.add_argument("--out", default="")
    ap.add_argument("--media-root", default="", help="root of the materialised media tree, for a plan built from real records")
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
    llm = LLM(args.model, tensor_parallel_size=args.tp, max_model_len=8192, max_num_batched_tokens=8192, max_num_seqs=8,
              max_chunk_size=8192, kvcache_block_size=256, num_kvcache_blocks=args.pages, cpu_kv_cache_ratio=0.0,
              **VARIANTS[args.variant])
    if not llm.is_driver:
        llm.serve_forever()
        return
    session = OnlineServingSession(llm)
    sp = SamplingParams(temperature=0.0, max_tokens=args.max_tokens, ignore_eos=True)
    load_image = load_image or (lambda d: image_for(d, args.image_size))
    images = {g.group_id: [load_image(d) for d in g.media_digests] for g in plan.groups}

    def payload(r: wsp.PlannedRequest) -> dict:
        g = plan.groups[r.group_index]
        return {"type": "interleaved_images", "prompt": wsp.media_first_prompt(g.num_images, g.questions[r.question_index]),
                "images": images[g.group_id], "image_marker": wsp.IMAGE_MARKER}

    t0 = time.perf_counter()
    for r in plan.population:  # closed loop: one at a time
        session.run([OnlineRequest(r.request_key, 0.0, payload(r), sp)])
    population_s = time.perf_counter() - t0
    session.reset_metrics()
    result = session.run([OnlineRequest(r.request_key, r.arrival_offset_s, payload(r), sp) for r in plan.measured])
    summary = online_serving.summarize_online_run({
        "duration_s": result.duration_s, "requests": [r.to_record() for r in result.requests],
        "scheduler_metrics": llm.metrics_snapshot()["scheduler"]})
    prefix = llm.multimodal_prefix_cache_metadata()
    record = {
        "schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "online_working_set",
        "engine": "prism_infer_b200", "model": args.model, "data": "synthetic",
        "hardware": {"gpus": args.tp},
        "provenance": harness.provenance(),
        "config": {"variant": args.variant, "groups": args.groups, "questions": args.questions, "requests": args.requests,
                   "rate_per_s": args.rate, "alpha": args.alpha, "pages": args.pages, "page_tokens": 256, "images_per_group": [args.min_images, args.max_images],
                   "kv_budget_bytes": args.pages * llm.config.kv_bytes_per_page(), "working_set_pages": plan.working_set_pages,
                   "max_tokens": args.max_tokens, "seed": args.seed, "tp": args.tp, "plan_sha256": plan_sha256},
        "results": {
            "ttft_p50_ms": summary["ttft_ms"]["p50"], "ttft_p99_ms": summary["ttft_ms"]["p99"],
            "e2e_p50_ms": summary["e2e_ms"]["p50"], "e2e_p99_ms": summary["e2e_ms"]["p99"],
            "recomputed_prompt_tokens": summary["recomputed_prompt_tokens"], "prompt_tokens": summary["prompt_tokens"],
            "output_tokens_per_s": summary["output_tokens_per_s"], "completed": summary["requests"]["completed"],
            "duration_s": result.duration_s, "population_s": population_s,
            "resident_media": prefix["entries"], "prefix_evictions": prefix["evictions"], "prefix_hits": prefix["hits"],
            "resident_pages": prefix["resident_pages"], "media_cache": result.cache_counters,
        },
    }
    benchmark_schema.validate_benchmark_record(record)
    print(json.dumps(record["results"]), flush=True)
    if args.out:
        benchmark_schema.write_record(args.out, record)
    session.close()
    llm.exit()


if __name__ == "__main__":
    main()
