"""Time to first token of the headline request (N x 448x448 images + 32 tokens), with the
engine's profile regions broken out: host preprocessing, scheduling, input preparation,
vision tower, language prefill, sampling.  TTFT here is wall clock from ``add_prepared_image_request``
to the step that returns the first token, after one untimed request.

    python benchmarks/bench_ttft.py [--images 8] [--repeats 5] [--tp 1] [--out rec.json]

Long-context form: ``--text-tokens 16384 --chunk 2048`` times a text-only prompt of that many random tokens prefilled in
chunks (every chunk after the first attends over the paged cache); ``--paged-prefill-kernel mma`` selects the
page-reading mma.sync kernel instead of the gather + tcgen05 pair, ``both`` measures one after the other in one process
(one JSON line each).
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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--out", default="")
    ap.add_argument("--text-tokens", type=int, default=0, help="text-only prompt of this many tokens instead of images")
    ap.add_argument("--chunk", type=int, default=8192, help="prefill chunk size (tokens)")
    ap.add_argument("--paged-prefill-kernel", choices=["tc", "mma", "both"], default="tc")
    ap.add_argument("--vision-graph", action="store_true", help="replay the vision tower from a CUDA graph per grid shape")
    ap.add_argument("--cuda-profiler-range", action="store_true",
                    help="bracket the last timed request with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
    ap.add_argument("--device", default=None)
    ap.add_argument("--image-size", type=int, default=448)
    args = ap.parse_args(argv)
    import torch

    sync = torch.cuda.synchronize if torch.cuda.is_available() else (lambda: None)

    from prism_infer_b200 import ops

    kernels = ["tc", "mma"] if args.paged_prefill_kernel == "both" else [args.paged_prefill_kernel]
    long_text = args.text_tokens > 0
    max_len = max(4096, args.text_tokens + 256)
    llm = LLM(args.model, device=args.device, tensor_parallel_size=args.tp, max_model_len=max_len, kvcache_block_size=256,
              num_kvcache_blocks=max(64, 2 * (max_len // 256) + 2), compression_mode="scaled_fp8_kv", max_num_seqs=4,
              max_num_batched_tokens=min(16384, args.chunk) if long_text else 16384, max_chunk_size=args.chunk,
              cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, enable_vision_tensor_cudagraph=args.vision_graph)
    if not llm.is_driver:
        llm.serve_forever()
        return
    rng = np.random.default_rng(0)
    proc = PatchProcessor(llm.arch)
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)

    vocab = min(150000, llm.arch.text.vocab_size - 64)  # below the special tokens of the model's vocabulary

    def make():
        t0 = time.perf_counter()
        if long_text:
            return rng.integers(0, vocab, args.text_tokens).tolist(), (time.perf_counter() - t0) * 1e3
        inp = prepare_image_inputs(proc, llm.tokenizer, rng.integers(0, vocab, 32).tolist(),
                                   [rng.integers(0, 256, (args.image_size, args.image_size, 3), dtype=np.uint8) for _ in range(args.images)])
        return inp, (time.perf_counter() - t0) * 1e3

    def one(inp) -> float:
        sync()
        t0 = time.perf_counter()
        if long_text:
            llm.add_request(inp, sp)
        else:
            llm.add_prepared_image_request(inp, sp)
        while not llm.is_finished():
            llm.step_result()
        sync()
        return (time.perf_counter() - t0) * 1e3

    for kernel in kernels:
        ops.PAGED_PREFILL_TC_ENABLED = kernel == "tc"
        one(make()[0])
        if not long_text:
            one(make()[0])
        ttft, prep = [], []
        workload = f"text{args.text_tokens}_chunk{args.chunk}_{kernel}" if long_text else f"images{args.images}"
        with performance_profile({"workload": workload, "tp": args.tp}, nvtx=False) as session:
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
        out = {"workload": workload, "tp": args.tp, "prompt_tokens": len(inp if long_text else inp.input_ids), "ttft_ms": [round(t, 2) for t in ttft],
               "ttft_median_ms": round(sorted(ttft)[n // 2], 2), "ttft_p50_ms": round(float(np.percentile(ttft, 50)), 2),
               "ttft_p99_ms": round(float(np.percentile(ttft, 99)), 2), "preprocess_ms_median": round(sorted(prep)[n // 2], 2), "regions": table}
        print(json.dumps(out), flush=True)
        if args.out:
            with open(args.out if len(kernels) == 1 else f"{args.out}.{kernel}", "w") as fh:
                json.dump(out, fh, indent=1)
    llm.exit()


if __name__ == "__main__":
    main()
