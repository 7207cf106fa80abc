"""Headline benchmark: Qwen3-VL-8B decode TPOT (ms per output token) on synthetic inputs.

Workload (the reference's headline config): random-init Qwen3-VL-8B weights, bf16 compute,
scaled-FP8 paged KV with 256-token pages, CUDA-graph decode, one request of 8 uniform-random
448x448 images (1568 visual tokens) plus a 32-token random question, batch 1, greedy.  With
``--gpus N`` the same request runs tensor-parallel over N GPUs (strong scaling).

``value`` / ``ms_per_step``: device time of one decode step, CUDA events around K
back-to-back launches of the engine's own decode graph (staging copy, 36 layers, LM head,
sampler, token copy-back), max over ranks.  A step streams ~15 GB of weights, far more than
the 126 MB L2, so no flush is needed between steps.
``e2e``: the same K steps through the public API (``LLM.step_result``): host scheduling,
filling the pinned staging buffer, the host-to-device copy of the step's inputs, the
device-to-host token read, per step (on one GPU the engine launches the next greedy step before
it waits for the current one, so host work overlaps device work).  ``first_tokens`` / ``first_tokens_sha1``: the first eight
generated token ids of the request, so that runs at different N can be compared by eye.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_TPOT_MS = 9.8821  # reference, RTX 5090, TP1, 8 x 448x448 images (docs/RESULTS.md:116)
PUBLISHED_TP2_TPOT_MS = 5.9701


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_reference(args) -> None:
    """The unmodified reference from baseline/_ref through its own public API."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
    except Exception as exc:  # pragma: no cover
        print(json.dumps({"impl": "reference", "unavailable": f"cannot import baseline/reference_arm.py: {exc}"}))
        return
    reference_arm.main(args)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="prism_b200")
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--kv-pages", type=int, default=0)
    ap.add_argument("--logits-precision", default="", choices=["", "model", "fp32", "selective_fp32"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import numpy as np
    import torch

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.engine.contracts import Phase
    from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs
    from prism_infer_b200.ops import native
    from prism_infer_b200.parallel.tp_group import rank_info

    rank, world = rank_info()
    if world > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    W, K = max(3, args.warmup), args.steps
    pages = args.kv_pages or max(16, args.batch * 12)
    # the reference's own tuned mode for this workload ranks greedy tokens with ``selective_fp32`` logits (FP8 candidate
    # head + exact rerank) on one GPU and requires the plain head under tensor parallelism; so does this arm
    logits_precision = args.logits_precision or ("selective_fp32" if args.gpus == 1 else "model")
    llm = LLM(args.model, tensor_parallel_size=args.gpus, max_model_len=4096, kvcache_block_size=256,
              num_kvcache_blocks=pages, compression_mode="scaled_fp8_kv", max_num_seqs=max(args.batch, 1),
              max_num_batched_tokens=16384, max_chunk_size=8192, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False,
              logits_precision=logits_precision)
    if not llm.is_driver:
        llm.serve_forever()  # tensor-parallel worker rank: follows rank 0 until shutdown
        return
    arch = llm.arch
    rng = np.random.default_rng(0)
    proc = PatchProcessor(arch)
    sp = SamplingParams(temperature=0.0, max_tokens=W + K + 2, ignore_eos=True)
    # one untimed request first: lazy initialisation (tensor maps, NCCL communicators, IPC
    # mappings, allocator pools) must not count towards TTFT
    warm = prepare_image_inputs(proc, llm.tokenizer, rng.integers(0, 150000, 32).tolist(),
                                [rng.integers(0, 256, (448, 448, 3), dtype=np.uint8) for _ in range(args.images)])
    llm.generate_prepared_image_inputs(warm, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    for b in range(args.batch):
        images = [rng.integers(0, 256, (448, 448, 3), dtype=np.uint8) for _ in range(args.images)]
        question = rng.integers(0, 150000, 32).tolist()
        inputs = prepare_image_inputs(proc, llm.tokenizer, question, images)
        llm.add_prepared_image_request(inputs, sp)
    prompt_tokens = len(inputs.input_ids)
    t_pre = time.perf_counter()
    while True:  # prefill (TTFT)
        res = llm.step_result()
        if res.phase is Phase.DECODE or llm.scheduler.num_decoding == args.batch:
            break
    torch.cuda.synchronize()
    ttft_ms = (time.perf_counter() - t_pre) * 1e3
    for _ in range(W):
        llm.step_result()
    torch.cuda.synchronize()

    # ---- e2e: K steps through the public API ------------------------------------------
    meta = llm.graph_metadata()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    llm.barrier()  # every rank's device idle before the timed region
    native.reset_launch_count()
    t0 = time.perf_counter()
    for _ in range(K):
        llm.step_result()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / K
    # the first generated tokens of the last request: the same at every N when tensor parallelism is exact enough
    running = list(llm._sequences.values())
    first_tokens = [int(t) for t in running[-1].completion_token_ids[:8]] if running else []
    # ---- device time: K back-to-back launches of the same decode graph ------------------
    device_ms = llm.time_decode_graph(K)  # maximum over ranks
    clocks = sampler.stop()
    launches = int(meta.get("launches_per_decode_graph", {}).get(str(max(1, args.batch)), 0)) * K
    stage_bytes = int(meta.get("staging_bytes", {}).get(str(max(1, args.batch)), 0))
    out = {
        "metric": "qwen3_vl_8b_decode_tpot_ms", "value": round(device_ms, 4), "unit": "ms/token",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": round(device_ms, 4),
        "higher_is_better": False, "scaling": "strong",
        "vs_baseline": round(device_ms / (PUBLISHED_TPOT_MS if args.gpus == 1 else PUBLISHED_TP2_TPOT_MS), 4),
        "dtype": "bf16", "data": "synthetic (uniform-random images and token ids, random-init weights)",
        "impl": "prism_b200",
        "config": {"model": "Qwen3-VL-8B (random init)", "global_batch": args.batch, "seq_len": prompt_tokens,
                   "images": f"{args.images}x448x448", "output_tokens": W + K + 2, "kv": "scaled_fp8 e4m3 + fp32 scale, 256-token pages",
                   "parallelism": f"tp{args.gpus}", "decode": "cuda_graph", "logits_precision": logits_precision,
                   "l2": "inputs larger than L2 (a step streams the bf16 weights, ~15 GB/tp)"},
        "output_tok_per_s": round(args.batch * 1e3 / device_ms, 2),
        "ttft_ms": round(ttft_ms, 2),
        "e2e": {"value": round(e2e_ms, 4), "unit": "ms/token", "h2d_bytes_per_step": stage_bytes,
                "d2h_bytes_per_step": 8 * max(1, args.batch), "output_tok_per_s": round(args.batch * 1e3 / e2e_ms, 2)},
        "gpu_launches": launches,
        "clocks": clocks,
        "first_tokens": first_tokens,
        "first_tokens_sha1": hashlib.sha1(",".join(map(str, first_tokens)).encode()).hexdigest()[:12],
    }
    print(json.dumps(out), flush=True)
    llm.exit()


if __name__ == "__main__":
    main()
