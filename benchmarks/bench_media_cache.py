"""Content-reuse benchmark: one manifest case expanded to a batch, with an exact fraction of the
requests carrying byte-identical media (reference ``benchmarks/multimodal_cache_workload.py`` as
used by its online and system runners).

Repeated media arrive in fresh arrays, so only content addressing (the visual-embedding cache and
the multimodal prefix cache, both keyed by SHA-256 of the pixels) can recognise them; every
non-repeated request gets a unique 64-bit marker in its first frame.  One record per repeat
rate: wall time for the batch through ``LLM.generate_mixed``, the caches' hit / miss counters,
(a visual-embedding miss is one run of the vision tower: requests are encoded at submission and
their prefill then reads the stored embedding, so misses, not hits, count the encoder work),
the peak device memory of the process, and the provenance block (source tree digest, GPU).

    python benchmarks/bench_media_cache.py [--case single_image_448] [--batch 16] [--repeat-rates 0 0.5 1] [--vary-questions] [--out rec.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Any, Sequence

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

import harness  # noqa: E402

from prism_infer_b200 import LLM, SamplingParams  # noqa: E402
from prism_infer_b200.analysis import benchmark_schema  # noqa: E402


def run_rates(llm, case: dict[str, Any], batch: int, rates: Sequence[float], *, vary_questions: bool, max_tokens: int,
              device_index: int = 0, nvml: Any = None) -> list[dict[str, Any]]:
    expanded, source, factor = harness.expand_case_batch(case, batch)
    base = harness.materialize_requests(expanded)
    sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
    out = []
    for rate in rates:
        payloads, reuse = harness.build_multimodal_cache_workload(base, repeat_rate=rate, vary_questions=vary_questions)
        vis0, pre0 = llm.visual_embedding_cache_metadata(), llm.multimodal_prefix_cache_metadata()
        with harness.GpuMemorySampler(device_index, nvml=nvml) as mem:
            t0 = time.perf_counter()
            results = llm.generate_mixed(payloads, sp, use_tqdm=False)
            wall = time.perf_counter() - t0
        vis1, pre1 = llm.visual_embedding_cache_metadata(), llm.multimodal_prefix_cache_metadata()
        delta = lambda a, b, k: int(b.get(k, 0)) - int(a.get(k, 0))  # noqa: E731
        out.append({
            "repeat_rate": rate, "reuse": reuse, "requests": len(payloads), "source_requests": source, "replication": factor,
            "wall_s": wall, "requests_per_s": len(payloads) / wall, "output_tokens": sum(len(r["token_ids"]) for r in results),
            "visual_embedding_cache": {k: delta(vis0, vis1, k) for k in ("hits", "misses")},
            "prefix_cache": {k: delta(pre0, pre1, k) for k in ("hits", "misses", "stores", "evictions")},
            "process_gpu_memory": mem.to_record(),
        })
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--manifest", default=os.path.join(ROOT, "benchmarks", "workloads", "system_cases.json"))
    ap.add_argument("--case", default="single_image_448")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--repeat-rates", type=float, nargs="*", default=[0.0, 0.5, 1.0])
    ap.add_argument("--vary-questions", action="store_true")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--mode", default="scaled_fp8_kv")
    ap.add_argument("--pages", type=int, default=512)
    ap.add_argument("--device", default=None)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    case = harness.find_workload_case(harness.load_manifest(args.manifest), args.case)
    llm = LLM(args.model, device=args.device, max_model_len=8192, kvcache_block_size=256, num_kvcache_blocks=args.pages, max_num_seqs=max(8, args.batch),
              max_num_batched_tokens=16384, max_chunk_size=8192, cpu_kv_cache_ratio=0.0, enable_prefix_caching=True,
              enable_visual_embedding_cache=True, compression_mode=args.mode)
    try:
        cells = run_rates(llm, case, args.batch, args.repeat_rates, vary_questions=args.vary_questions, max_tokens=args.max_tokens)
    finally:
        llm.exit()
    record = {"schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "media_cache_reuse", "engine": "prism_infer_b200",
              "model": args.model, "data": "synthetic", "hardware": {"gpus": 1},
              "config": {"case": args.case, "batch": args.batch, "mode": args.mode, "vary_questions": args.vary_questions,
                         "max_tokens": args.max_tokens, "inputs": harness.describe_case_inputs(case)},
              "results": {"cells": cells}, "provenance": harness.provenance()}
    benchmark_schema.validate_benchmark_record(record)
    for c in cells:
        print(json.dumps({"repeat_rate": c["repeat_rate"], "wall_s": round(c["wall_s"], 4), "visual": c["visual_embedding_cache"],
                          "prefix": c["prefix_cache"]}), flush=True)
    if args.out:
        benchmark_schema.write_record(args.out, record)


if __name__ == "__main__":
    main()
