"""Mode matrix: every execution / compression mode against named synthetic workloads, one
record per (mode, workload) with TTFT, TPOT, end-to-end latency and output tokens/s (mirrors
the reference's ``benchmarks/bench_system.py:77-316`` and ``bench_vl_cudagraph_decode.py``:
eager against CUDA-graph decode, BF16 against FP8 / scaled-FP8 KV, dense against compacted
visual context).

    python benchmarks/bench_system.py [--modes eager graph ...] [--workloads single_image_448 ...]
                                      [--tensor-parallel-size N] [--batch 1] [--out records.json]
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


def run_cell(llm, wl: dict, batch: int, rng) -> dict:
    sp = SamplingParams(temperature=0.0, max_tokens=wl["output_tokens"], ignore_eos=True)

    def submit():
        req = build_request(llm, wl, rng)
        if isinstance(req, list):
            llm.add_request(req, sp)
        elif wl["kind"] == "video":
            llm.add_prepared_video_request(req, sp)
        else:
            llm.add_prepared_image_request(req, sp)

    submit()                      # untimed: lazy initialisation
    while not llm.is_finished():
        llm.step_result()
    for _ in range(batch):
        submit()
    t0 = time.perf_counter()
    first = None
    tokens = 0
    while not llm.is_finished():
        res = llm.step_result()
        tokens += len(res.outputs) if hasattr(res, "outputs") else 0
        if first is None and llm.scheduler.num_decoding == batch:
            first = time.perf_counter()
    t1 = time.perf_counter()
    n_out = wl["output_tokens"]
    ttft = ((first or t1) - t0) * 1e3
    tpot = (t1 - (first or t0)) * 1e3 / max(1, n_out - 1)
    return {"ttft_ms": ttft, "tpot_ms": tpot, "e2e_ms": (t1 - t0) * 1e3, "output_tokens_per_s": batch * n_out / (t1 - t0),
            "batch": batch}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--modes", nargs="*", default=["eager", "graph", "graph_scaled_fp8_kv", "graph_visual_compact_scaled_fp8"])
    ap.add_argument("--workloads", nargs="*", default=["single_image_448", "eight_image_448"])
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    records = []
    provenance = harness.provenance()
    for mode in args.modes:
        if mode not in MODES:
            raise SystemExit(f"unknown mode {mode!r}; known: {sorted(MODES)}")
        opts = dict(MODES[mode])
        llm = LLM(args.model, tensor_parallel_size=args.tensor_parallel_size, max_model_len=args.max_model_len, kvcache_block_size=256,
                  num_kvcache_blocks=max(64, args.batch * 24), max_num_seqs=max(args.batch, 1), max_num_batched_tokens=16384,
                  max_chunk_size=8192, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, **opts)
        if not llm.is_driver:
            llm.serve_forever()
            continue
        rng = np.random.default_rng(0)
        for name in args.workloads:
            wl = load_workload(name)
            res = run_cell(llm, wl, args.batch, rng)
            rec = {"schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "system_mode_matrix", "engine": "prism_infer_b200",
                   "model": args.model, "data": "synthetic", "hardware": {"gpus": args.tensor_parallel_size},
                   "config": {"mode": mode, "workload": name, **{k: v for k, v in opts.items()}, "tp": args.tensor_parallel_size},
                   "results": res, "provenance": provenance}
            benchmark_schema.validate_benchmark_record(rec)
            records.append(rec)
            print(json.dumps({"mode": mode, "workload": name, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in res.items()}}), flush=True)
        llm.exit()
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(records, fh, indent=1)


if __name__ == "__main__":
    main()
