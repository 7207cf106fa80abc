"""Decode / prefill latency matrix on synthetic inputs: TTFT, TPOT, output tokens/s for a
grid of (workload, batch size) at a given tensor-parallel size.  Workloads: ``images8`` (8 x
448x448 images + 32 tokens), ``image1`` (1 image + 32 tokens), ``video16`` (16-frame 448x448
clip + 32 tokens, chunked prefill 2048), ``text`` (256 random tokens).  Mirrors the
reference's ``benchmarks/bench_external_prism.py`` / ``bench_system.py`` metrics: TTFT = first
token time after preprocessing, TPOT = (last - first token time) / (n - 1).  At larger batches that TPOT contains the prefill batches of the
other requests; ``steady_step_ms_median`` is the wall time of a decode step in which every sequence of the batch
decodes.

    python benchmarks/bench_decode.py --workload image1 --batches 1,8,32,128 [--tp 8] [--out rec.json]
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
from prism_infer_b200.analysis import benchmark_schema  # noqa: E402
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs, prepare_video_inputs  # noqa: E402


def token_ids(llm, rng, n: int) -> list[int]:
    """Random ids below the special tokens of the model's vocabulary."""
    return rng.integers(0, min(150000, llm.arch.text.vocab_size - 64), n).tolist()


def build_inputs(llm, workload: str, rng, size: int = 448):
    proc = PatchProcessor(llm.arch)
    q = token_ids(llm, rng, 32)
    picture = lambda: rng.integers(0, 256, (size, size, 3), dtype=np.uint8)  # noqa: E731
    if workload == "images8":
        return prepare_image_inputs(proc, llm.tokenizer, q, [picture() for _ in range(8)])
    if workload == "image1":
        return prepare_image_inputs(proc, llm.tokenizer, q, [picture()])
    if workload == "video16":
        return prepare_video_inputs(proc, llm.tokenizer, q, [picture() for _ in range(16)])
    return None


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--workload", default="image1", choices=["images8", "image1", "video16", "text"])
    ap.add_argument("--batches", default="1,8,32,128")
    ap.add_argument("--output-tokens", type=int, default=128)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--out", default="")
    ap.add_argument("--device", default=None)
    ap.add_argument("--image-size", type=int, default=448)
    ap.add_argument("--text-tokens", type=int, default=256, help="prompt length of the text workload")
    args = ap.parse_args(argv)
    batches = [int(b) for b in args.batches.split(",")]
    llm = LLM(args.model, device=args.device, tensor_parallel_size=args.tp, max_model_len=4096, kvcache_block_size=256,
              num_kvcache_blocks=max(64, max(batches) * 10), compression_mode="scaled_fp8_kv", max_num_seqs=max(batches),
              max_num_batched_tokens=16384, max_chunk_size=args.chunk, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False)
    if not llm.is_driver:
        llm.serve_forever()
        return
    rng = np.random.default_rng(0)
    sp = SamplingParams(temperature=0.0, max_tokens=args.output_tokens, ignore_eos=True)
    rows = []
    for b in batches:
        for rep in range(2):  # first repetition warms up
            ids = []
            t_submit = time.perf_counter()
            for _ in range(b):
                inp = build_inputs(llm, args.workload, rng, args.image_size)
                if inp is None:
                    ids.append(llm.add_request(token_ids(llm, rng, args.text_tokens), sp))
                elif args.workload == "video16":
                    ids.append(llm.add_prepared_video_request(inp, sp))
                else:
                    ids.append(llm.add_prepared_image_request(inp, sp))
            t_ready = time.perf_counter()
            first: dict[int, float] = {}
            last: dict[int, float] = {}
            count: dict[int, int] = {}
            steady: list[float] = []  # wall time of decode steps in which all b sequences decode
            while not llm.is_finished():
                full = llm.scheduler.num_decoding == b
                t_step = time.perf_counter()
                res = llm.step_result()
                now = time.perf_counter()
                if full and res.phase.value == "decode" and len(res.outputs) == b:
                    steady.append((now - t_step) * 1e3)
                for o in res.outputs:
                    if o.new_token is not None:
                        first.setdefault(o.request_id, now)
                        last[o.request_id] = now
                        count[o.request_id] = count.get(o.request_id, 0) + 1
            t_end = time.perf_counter()
        ttft = [(first[i] - t_ready) * 1e3 for i in ids]
        tpot = [(last[i] - first[i]) * 1e3 / max(1, count[i] - 1) for i in ids]
        row = {"batch": b, "ttft_ms_mean": float(np.mean(ttft)), "ttft_ms_max": float(np.max(ttft)),
               "tpot_ms_mean": float(np.mean(tpot)), "output_tok_per_s": b * args.output_tokens / (t_end - t_ready),
               "preprocess_ms": (t_ready - t_submit) * 1e3}
        if len(steady) > 8:  # per-step figures without the other requests' prefill batches in between
            core = sorted(steady[4:])
            row["steady_step_ms_median"] = float(core[len(core) // 2])
            row["steady_tok_per_s"] = b * 1e3 / row["steady_step_ms_median"]
        rows.append(row)
        print(json.dumps(row), flush=True)
    record = {"schema_version": benchmark_schema.BENCHMARK_SCHEMA_VERSION, "benchmark": "decode_matrix",
              "engine": "prism_infer_b200", "model": args.model, "data": "synthetic", "hardware": {"gpus": args.tp},
              "config": {"workload": args.workload, "output_tokens": args.output_tokens, "tp": args.tp, "chunk": args.chunk,
                         "kv": "scaled_fp8"},
              "results": {"rows": rows}}
    benchmark_schema.validate_benchmark_record(record)
    if args.out:
        benchmark_schema.write_record(args.out, record)
    llm.exit()


if __name__ == "__main__":
    main()
