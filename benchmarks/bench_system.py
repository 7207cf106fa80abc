"""Mode matrix: every execution / compression mode against named synthetic workloads, one
record per (mode, workload) with TTFT, TPOT, end-to-end latency and output tokens/s (mirrors
the reference's ``benchmarks/bench_system.py:77-316`` and ``bench_vl_cudagraph_decode.py``:
eager against CUDA-graph decode, BF16 against FP8 / scaled-FP8 KV, dense against compacted
visual context).

    python benchmarks/bench_system.py [--modes eager graph ...] [--workloads single_image_448 ...]
                                      [--tensor-parallel-size N] [--batch-sizes 1 8] [--output-lengths 32 128]
                                      [--visual-pruning-keep-ratios 0.4 0.6] [--profile-output prof.json] [--out records.json]

Batch sizes and output lengths are swept inside one engine per mode; keep ratios (compacting and pruning modes only) get
an engine each.  ``--profile-output`` writes the performance profile of the last timed cell.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

import harness  # noqa: E402

from prism_infer_b200 import LLM, SamplingParams  # noqa: E402
from prism_infer_b200.analysis import benchmark_schema  # noqa: E402
from prism_infer_b200.analysis.identity import canonical_json_sha256  # noqa: E402
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs, prepare_video_inputs  # noqa: E402

MODES = {
    "eager": dict(enforce_eager=True, compression_mode="off"),
    "graph": dict(enforce_eager=False, compression_mode="off"),
    "graph_fp8_kv": dict(enforce_eager=False, compression_mode="fp8_kv"),
    "graph_scaled_fp8_kv": dict(enforce_eager=False, compression_mode="scaled_fp8_kv"),
    "eager_scaled_fp8_kv": dict(enforce_eager=True, compression_mode="scaled_fp8_kv"),
    "graph_visual_compact": dict(enforce_eager=False, compression_mode="visual_compact", visual_pruning_keep_ratio=0.6),
    "graph_visual_compact_scaled_fp8": dict(enforce_eager=False, compression_mode="visual_compact_scaled_fp8",
                                            visual_pruning_keep_ratio=0.6),
    "eager_visual_prune": dict(enforce_eager=True, compression_mode="visual_prune", visual_pruning_keep_ratio=0.6),
}


def load_workload(name: str) -> dict:
    with open(os.path.join(ROOT, "benchmarks", "workloads", name + ".json")) as fh:
        return json.load(fh)


def build_request(llm, wl: dict, rng):
    proc = PatchProcessor(llm.arch)
    vocab = min(150000, llm.arch.text.vocab_size - 64)
    q = rng.integers(0, vocab, wl["question_tokens"]).tolist()
    size = wl["image_size"]
    if wl["kind"] in ("image", "images"):
        return prepare_image_inputs(proc, llm.tokenizer, q, [rng.integers(0, 256, (size, size, 3), dtype=np.uint8) for _ in range(wl["images"])])
    if wl["kind"] == "video":
        return prepare_video_inputs(proc, llm.tokenizer, q, [rng.integers(0, 256, (size, size, 3), dtype=np.uint8) for _ in range(wl["frames"])])
    return q


STAT_KEYS = ("count", "median", "p90", "p99", "min", "max")


def summarize(values) -> dict:
    """count / median / p90 / p99 / min / max with linear interpolation between order statistics."""
    v = np.sort(np.asarray(list(values), dtype=np.float64))
    if v.size == 0:
        raise ValueError("no values to summarise")
    return {"count": int(v.size), "median": float(np.percentile(v, 50)), "p90": float(np.percentile(v, 90)),
            "p99": float(np.percentile(v, 99)), "min": float(v[0]), "max": float(v[-1])}


def _graph_meta(llm) -> dict:
    meta = llm.graph_metadata()
    return meta[0] if isinstance(meta, (list, tuple)) else meta


def _counts(meta: dict) -> dict[str, dict[int, int]]:
    steps = meta.get("decode_steps", {})
    return {k: {int(n): int(c) for n, c in steps.get(k, {}).items()} for k in ("graph_batch_sizes", "eager_batch_sizes")}


def run_cell(llm, wl: dict, batch: int, rng, *, repeats: int = 1) -> dict:
    """``repeats`` timed rounds of ``batch`` identical-shape requests after one untimed request.  Returns the
    latency statistics, which path every decode step took (graph replay per bucket or eager), the token ids of
    every request and the KV accounting of the prompts."""
    sp = SamplingParams(temperature=0.0, max_tokens=wl["output_tokens"], ignore_eos=True)

    def submit(req) -> int:
        if isinstance(req, list):
            return llm.add_request(req, sp)
        if wl["kind"] == "video":
            return llm.add_prepared_video_request(req, sp)
        return llm.add_prepared_image_request(req, sp)

    submit(build_request(llm, wl, rng))  # untimed: lazy initialisation
    while not llm.is_finished():
        llm.step_result()
    requests = [build_request(llm, wl, rng) for _ in range(batch)]  # the same inputs every round: token ids must repeat
    n_out = wl["output_tokens"]
    ttft, tpot, e2e, rate = [], [], [], []
    rounds_tokens: list[list[list[int]]] = []
    llm.reset_metrics()
    before = _counts(_graph_meta(llm))
    for _ in range(repeats):
        ids = [submit(r) for r in requests]
        done: dict[int, list[int]] = {}
        t0 = time.perf_counter()
        first = None
        while not llm.is_finished():
            res = llm.step_result()
            for o in res.outputs:
                if o.finished:
                    done[o.request_id] = [int(t) for t in o.token_ids]
            if first is None and llm.scheduler.num_decoding + len(done) == batch:
                first = time.perf_counter()
        t1 = time.perf_counter()
        ttft.append(((first or t1) - t0) * 1e3)
        tpot.append((t1 - (first or t0)) * 1e3 / max(1, n_out - 1))
        e2e.append((t1 - t0) * 1e3)
        rate.append(batch * n_out / (t1 - t0))
        rounds_tokens.append([done[i] for i in ids])
    after = _counts(_graph_meta(llm))
    meta = _graph_meta(llm)
    snap = llm.metrics_snapshot()["engine"]
    decode_sizes: dict[int, int] = {}
    for bt in snap["batches"]:
        if bt["phase"] == "decode":
            decode_sizes[int(bt["batch_size"])] = decode_sizes.get(int(bt["batch_size"]), 0) + 1
    delta = {k: {n: c - before[k].get(n, 0) for n, c in after[k].items() if c - before[k].get(n, 0)} for k in after}
    buckets = sorted(int(x) for x in meta.get("buckets", []))
    replays = {b: 0 for b in buckets}
    for n, c in delta["graph_batch_sizes"].items():
        replays[next(b for b in buckets if b >= n)] += c
    page = int(llm.config.kvcache_block_size)
    per_page = int(meta.get("kv_bytes_per_page") or llm.config.kv_bytes_per_page())
    reqs = snap["requests"][-batch:]
    prompt = [int(r["prompt_tokens"]) for r in reqs]
    dropped = [int(r.get("dropped_prompt_tokens", 0)) for r in reqs]
    pages = lambda n: -(-n // page)  # noqa: E731
    stats = {"ttft_ms": summarize(ttft), "tpot_ms": summarize(tpot), "e2e_ms": summarize(e2e), "output_tokens_per_s": summarize(rate)}
    return {
        "results": {"ttft_ms": stats["ttft_ms"]["median"], "tpot_ms": stats["tpot_ms"]["median"], "e2e_ms": stats["e2e_ms"]["median"],
                    "output_tokens_per_s": stats["output_tokens_per_s"]["median"], "batch": batch, "stats": stats},
        "execution": {"backend": "cuda_graph" if buckets else "eager", "graph_batch_sizes": buckets,
                      "decode_batch_sizes": {str(n): c for n, c in sorted(decode_sizes.items())},
                      "graph_replays": {str(b): c for b, c in replays.items()},
                      "eager_decode_steps": sum(delta["eager_batch_sizes"].values()),
                      "decode_steps": sum(decode_sizes.values()), "run_ahead": dict(meta.get("decode_run_ahead", {}))},
        "correctness": {"requests": batch, "output_tokens": n_out, "output_token_ids": rounds_tokens[0],
                        "output_token_ids_sha256": canonical_json_sha256(rounds_tokens[0]),
                        "identical_across_repeats": all(r == rounds_tokens[0] for r in rounds_tokens)},
        "kv_cache": {"mode": llm.config.prism.cache.compression_mode, "kv_mode": int(llm.config.kv_mode), "page_tokens": page, "pages": int(meta.get("kv_pages", 0)),
                     "bytes_per_page": per_page, "prompt_tokens": prompt, "dropped_prompt_tokens": dropped,
                     "dense_prompt_bytes": sum(pages(n) for n in prompt) * per_page,
                     "active_prompt_bytes": sum(pages(n - d) for n, d in zip(prompt, dropped)) * per_page},
    }


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--modes", nargs="*", default=["eager", "graph", "graph_scaled_fp8_kv", "graph_visual_compact_scaled_fp8"])
    ap.add_argument("--workloads", nargs="*", default=["single_image_448", "eight_image_448"])
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--batch-sizes", type=int, nargs="*", default=None, help="sweep; overrides --batch")
    ap.add_argument("--output-lengths", type=int, nargs="*", default=None, help="sweep of output tokens; default: the workload's own")
    ap.add_argument("--visual-pruning-keep-ratios", type=float, nargs="*", default=None, help="sweep for modes that drop visual tokens")
    ap.add_argument("--profile-output", default="")
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--repeats", type=int, default=3, help="timed rounds per (mode, workload)")
    ap.add_argument("--device", default=None)
    ap.add_argument("--page-tokens", type=int, default=256)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    records = []
    provenance = harness.provenance()
    batches = args.batch_sizes or [args.batch]
    profile = None
    for mode in args.modes:
        if mode not in MODES:
            raise SystemExit(f"unknown mode {mode!r}; known: {sorted(MODES)}")
        ratios = args.visual_pruning_keep_ratios if (args.visual_pruning_keep_ratios and "visual_pruning_keep_ratio" in MODES[mode]) else [None]
        for ratio in ratios:
            opts = dict(MODES[mode])
            if ratio is not None:
                opts["visual_pruning_keep_ratio"] = ratio
            llm = LLM(args.model, device=args.device, tensor_parallel_size=args.tensor_parallel_size, max_model_len=args.max_model_len,
                      kvcache_block_size=args.page_tokens,
                      num_kvcache_blocks=max(64, max(batches) * 24), max_num_seqs=max(max(batches), 1), max_num_batched_tokens=16384,
                      max_chunk_size=8192, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, **opts)
            if not llm.is_driver:
                llm.serve_forever()
                continue
            rng = np.random.default_rng(0)
            for name in args.workloads:
                for n_out in (args.output_lengths or [None]):
                    wl = load_workload(name)
                    if n_out is not None:
                        wl["output_tokens"] = n_out
                    for batch in batches:
                        if args.profile_output:
                            from prism_infer_b200.analysis.performance_profile import performance_profile

                            with performance_profile({"mode": mode, "workload": name, "batch": batch}, nvtx=False) as session:
                                cell = run_cell(llm, wl, batch, rng, repeats=args.repeats)
                            profile = session.finalize()
                        else:
                            cell = run_cell(llm, wl, batch, rng, repeats=args.repeats)
                        res = cell["results"]
                        rec = {"schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "system_mode_matrix",
                               "engine": "prism_infer_b200", "model": args.model, "data": "synthetic", "hardware": {"gpus": args.tensor_parallel_size},
                               "config": {"mode": mode, "workload": name, **{k: v for k, v in opts.items()}, "tp": args.tensor_parallel_size,
                                          "repeats": args.repeats, "output_tokens": wl["output_tokens"]},
                               "results": res, "execution": cell["execution"], "correctness": cell["correctness"], "kv_cache": cell["kv_cache"],
                               "provenance": provenance}
                        benchmark_schema.validate_benchmark_record(rec)
                        records.append(rec)
                        if not args.quiet:
                            print(json.dumps({"mode": mode, "workload": name, "keep_ratio": ratio, "output_tokens": wl["output_tokens"],
                                              **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in res.items() if k != "stats"},
                                              "graph_replays": cell["execution"]["graph_replays"],
                                              "eager_decode_steps": cell["execution"]["eager_decode_steps"]}), flush=True)
            llm.exit()
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(records, fh, indent=1)
    if args.profile_output and profile is not None:
        from prism_infer_b200.analysis.performance_profile import validate_profile_record

        with open(args.profile_output, "w") as fh:
            json.dump(validate_profile_record(profile), fh, indent=1)


if __name__ == "__main__":
    main()
