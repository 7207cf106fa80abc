"""KV capacity: bytes per page and token capacity for bf16, FP8 and scaled-FP8 pages at a byte budget (accounting; the
reference's ``bench_kv_capacity.py`` and ``docs/RESULTS.md:128-137``: 4 068.000 -> 2 097.562 MiB for 113 pages,
28 928 -> 56 320 tokens at about 4 GiB), and with ``--measure`` the capacity an engine actually reaches: for every mode
an engine whose page count is the budget divided by that mode's bytes per page gets ``--requests`` copies of a manifest
case at once, and the run reports how many sequences were resident at the peak, how many were preempted and how many
pages the prompts occupied.

    python benchmarks/bench_kv_capacity.py [--budget-bytes 4282122240] [--tp 1]
    python benchmarks/bench_kv_capacity.py --measure --case single_image_448 --requests 64 --max-tokens 16 [--modes off scaled_fp8_kv]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

from prism_infer_b200.config import Config  # noqa: E402

MODES = ("off", "fp8_kv", "scaled_fp8_kv", "visual_compact_scaled_fp8")


def accounting(model: str, budget_bytes: int, tp: int, page_tokens: int = 256, modes=("off", "fp8_kv", "scaled_fp8_kv")) -> dict:
    out = {}
    for mode in modes:
        cfg = Config(model, compression_mode=mode, tensor_parallel_size=tp, kvcache_block_size=page_tokens)
        per = cfg.kv_bytes_per_page() * tp
        pages = budget_bytes // per
        out[mode] = {"bytes_per_page": per, "pages": pages, "tokens": pages * page_tokens, "mib_for_113_pages": 113 * per / 2**20}
    if "off" in out and "scaled_fp8_kv" in out:
        out["scaled_over_bf16_bytes"] = out["scaled_fp8_kv"]["bytes_per_page"] / out["off"]["bytes_per_page"]
    return out


def measure(make_engine, case: dict, *, mode: str, pages: int, requests: int, max_tokens: int, manifest_dir: str | None = None) -> dict:
    """``requests`` copies of the case's first request, submitted together, on an engine with ``pages`` KV pages."""
    import harness

    from prism_infer_b200 import SamplingParams

    llm = make_engine(mode, pages)
    try:
        payload = harness.materialize_requests({"requests": case["requests"][:1]}, base=manifest_dir)[0]
        sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
        outs = llm.generate_mixed([dict(payload) for _ in range(requests)], sp, use_tqdm=False)
        counters = dict(llm.scheduler.counters)
        reqs = llm.metrics_snapshot()["engine"]["requests"][-requests:]
        page = llm.config.kvcache_block_size
        prompt_pages = [-(-(int(r["prompt_tokens"]) - int(r.get("dropped_prompt_tokens", 0))) // page) for r in reqs]
        return {"mode": mode, "pages": pages, "bytes_per_page": llm.config.kv_bytes_per_page(), "requests": requests,
                "completed": sum(len(o["token_ids"]) == max_tokens for o in outs), "peak_resident_sequences": counters.get("peak_running", 0),
                "preempted": counters.get("preempt_swap", 0) + counters.get("preempt_recompute", 0), "rejected": counters.get("rejected", 0),
                "prompt_pages_per_request": prompt_pages[0] if prompt_pages else 0,
                "sequences_that_fit_by_pages": pages // max(1, prompt_pages[0]) if prompt_pages else 0}
    finally:
        llm.exit()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--budget-bytes", type=int, default=4_282_122_240)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--page-tokens", type=int, default=256)
    ap.add_argument("--measure", action="store_true", help="run engines at the budget instead of only accounting")
    ap.add_argument("--modes", nargs="*", default=["off", "scaled_fp8_kv"], choices=MODES)
    ap.add_argument("--manifest", default=os.path.join(ROOT, "benchmarks", "workloads", "system_cases.json"))
    ap.add_argument("--case", default="single_image_448")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--device", default=None)
    ap.add_argument("--output", default="")
    args = ap.parse_args(argv)
    out = {"accounting": accounting(args.model, args.budget_bytes, args.tp, args.page_tokens)}
    if args.measure:
        import harness

        from prism_infer_b200 import LLM

        case = harness.find_workload_case(harness.load_manifest(args.manifest), args.case)
        per_mode = accounting(args.model, args.budget_bytes, args.tp, args.page_tokens, modes=args.modes)

        def make_engine(mode: str, pages: int):
            extra = dict(visual_pruning_keep_ratio=0.6) if mode.startswith("visual_compact") else {}
            return LLM(args.model, device=args.device, tensor_parallel_size=args.tp, compression_mode=mode, kvcache_block_size=args.page_tokens,
                       num_kvcache_blocks=pages, max_model_len=args.max_model_len, max_num_seqs=max(args.requests, 1),
                       max_num_batched_tokens=max(8192, args.max_model_len), max_chunk_size=max(8192, args.max_model_len),
                       cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, **extra)

        out["measured"] = [measure(make_engine, case, mode=m, pages=int(per_mode[m]["pages"]), requests=args.requests, max_tokens=args.max_tokens,
                                   manifest_dir=os.path.dirname(os.path.abspath(args.manifest))) for m in args.modes]
    print(json.dumps(out, indent=1))
    if args.output:
        with open(args.output, "w", encoding="utf-8") as fh:
            json.dump(out, fh, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
