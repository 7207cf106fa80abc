"""Time to first token of the headline request (N x 448x448 images + 32 tokens), with the
engine's profile regions broken out: host preprocessing, scheduling, input preparation,
vision tower, language prefill, sampling.  TTFT here is wall clock from ``add_prepared_image_request``
to the step that returns the first token, after one untimed request.

    python benchmarks/bench_ttft.py [--images 8] [--repeats 5] [--tp 1] [--out rec.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import LLM, SamplingParams  # noqa: E402
from prism_infer_b200.analysis.performance_profile import performance_profile  # noqa: E402
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--out", default="")
    ap.add_argument("--vision-graph", action="store_true", help="replay the vision tower from a CUDA graph per grid shape")
    ap.add_argument("--cuda-profiler-range", action="store_true",
                    help="bracket the last timed request with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    args = ap.parse_args()
    import torch

    sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)

    llm = LLM(args.model, tensor_parallel_size=args.tp, max_model_len=4096, kvcache_block_size=256, num_kvcache_blocks=64,
              compression_mode="scaled_fp8_kv", max_num_seqs=4, max_num_batched_tokens=16384, max_chunk_size=8192,
              cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, enable_vision_tensor_cudagraph=args.vision_graph)
    if not llm.is_driver:
        llm.serve_forever()
        return
    rng = np.random.default_rng(0)
    proc = PatchProcessor(llm.arch)
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)

    def make():
        t0 = time.perf_counter()
        inp = prepare_image_inputs(proc, llm.tokenizer, rng.integers(0, 150000, 32).tolist(),
                                   [rng.integers(0, 256, (448, 448, 3), dtype=np.uint8) for _ in range(args.images)])
        return inp, (time.perf_counter() - t0) * 1e3

    def one(inp) -> float:
        sync()
        t0 = time.perf_counter()
        llm.add_prepared_image_request(inp, sp)
        while not llm.is_finished():
            llm.step_result()
        sync()
        return (time.perf_counter() - t0) * 1e3

    one(make()[0])
    one(make()[0])
    ttft, prep = [], []
    with performance_profile({"workload": f"images{args.images}", "tp": args.tp}, nvtx=False) as session:
        for rep in range(args.repeats):
            inp, p = make()
            prep.append(p)
            ranged = args.cuda_profiler_range and rep == args.repeats - 1 and torch.cuda.is_available()
            if ranged:
                torch.cuda.profiler.start()
            ttft.append(one(inp))
            if ranged:
                torch.cuda.profiler.stop()
    rec = session.finalize()
    n = args.repeats
    table = {k: {"count_per_request": v["count"] / n, "cpu_ms": round(v["cpu_ms"] / n, 3), "cuda_ms": round(v["cuda_ms"] / n, 3)}
             for k, v in sorted(rec["totals"].items())}
    out = {"workload": f"images{args.images}", "tp": args.tp, "prompt_tokens": len(inp.input_ids), "ttft_ms": [round(t, 2) for t in ttft],
           "ttft_median_ms": round(sorted(ttft)[n // 2], 2), "ttft_p50_ms": round(float(np.percentile(ttft, 50)), 2),
           "ttft_p99_ms": round(float(np.percentile(ttft, 99)), 2), "preprocess_ms_median": round(sorted(prep)[n // 2], 2), "regions": table}
    print(json.dumps(out), flush=True)
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(out, fh, indent=1)
    llm.exit()


if __name__ == "__main__":
    main()
