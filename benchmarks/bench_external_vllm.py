"""The headline request on vLLM, for a same-box comparison with another engine (the reference ships
``benchmarks/bench_external_vllm.py`` for the same purpose).

The request is the one ``bench.py`` times: N uniform-noise 448 x 448 images and 32 random token ids, K output tokens,
greedy, random-init Qwen3-VL-8B weights written as a safetensors checkpoint with a synthetic tokenizer and processor
configuration (``baseline/reference_arm.write_checkpoint``; no download).  vLLM gets token-id prompts with one
``<|vision_start|><|image_pad|><|vision_end|>`` run per image and the images as ``multi_modal_data``; it expands the
placeholders itself.  Times are wall clock around ``LLM.generate``: TTFT from a run with one output token, TPOT as
``(t(K + 1 tokens) - t(1 token)) / K``, the definition the reference arm of ``bench.py`` uses.

    python benchmarks/bench_external_vllm.py [--images 8] [--output-tokens 64] [--tp 1] [--kv-cache-dtype fp8] [--out rec.json]

Prints one JSON line; ``{"engine": "vllm", "unavailable": "..."}`` when vLLM or a CUDA device is missing.  Not part of the
package's own execution path: vLLM is library code that is only driven here.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from typing import Any, Callable, Sequence

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def unavailable(why: str) -> dict[str, Any]:
    return {"engine": "vllm", "unavailable": " ".join(str(why).split())[:400]}


def build_prompt(arch, question_ids: Sequence[int], n_images: int) -> list[int]:
    """Media first, one placeholder per image (the engine under test expands it to the image's token count)."""
    ids: list[int] = []
    for _ in range(n_images):
        ids += [arch.vision_start_token_id, arch.image_token_id, arch.vision_end_token_id]
    return ids + [int(t) for t in question_ids]


def make_requests(arch, rng: np.random.Generator, *, batch: int, images: int, size: int, question_tokens: int) -> list[dict[str, Any]]:
    from PIL import Image

    vocab = min(150000, arch.text.vocab_size - 64)
    out = []
    for _ in range(batch):
        pics = [Image.fromarray(rng.integers(0, 256, (size, size, 3), dtype=np.uint8)) for _ in range(images)]
        prompt = {"prompt_token_ids": build_prompt(arch, rng.integers(0, vocab, question_tokens).tolist(), images)}
        if pics:
            prompt["multi_modal_data"] = {"image": pics}
        out.append(prompt)
    return out


def measure(generate: Callable[[list[dict[str, Any]], int], list[list[int]]], make: Callable[[], list[dict[str, Any]]], *,
            output_tokens: int, warmup: int, repeats: int, clock: Callable[[], float] = time.perf_counter) -> dict[str, Any]:
    """``generate(prompts, max_tokens) -> token ids per prompt``.  Every timed call gets fresh inputs, so no prefix or
    media cache of the engine under test shortens it."""
    for _ in range(warmup):
        generate(make(), 2)
    first, full, tokens = [], [], None
    for _ in range(repeats):
        t0 = clock()
        generate(make(), 1)
        first.append((clock() - t0) * 1e3)
        t0 = clock()
        out = generate(make(), output_tokens + 1)
        full.append((clock() - t0) * 1e3)
        if any(len(o) != output_tokens + 1 for o in out):
            raise RuntimeError(f"the engine returned {[len(o) for o in out]} tokens, {output_tokens + 1} asked for (is ignore_eos honoured?)")
        tokens = out
    ttft, e2e = float(np.median(first)), float(np.median(full))
    return {"ttft_ms": ttft, "tpot_ms": (e2e - ttft) / output_tokens, "e2e_ms": e2e, "ttft_ms_all": first, "e2e_ms_all": full,
            "first_tokens": [o[:8] for o in tokens or []]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--size", type=int, default=448)
    ap.add_argument("--question-tokens", type=int, default=32)
    ap.add_argument("--output-tokens", type=int, default=64)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--kv-cache-dtype", default="fp8", help="vLLM's kv_cache_dtype (auto, fp8, ...)")
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--checkpoint", default="", help="checkpoint directory; default: a random-init 8B one under the temp directory")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)
    try:
        import torch

        if not torch.cuda.is_available():
            print(json.dumps(unavailable("no CUDA device")))
            return 0
        import vllm
    except Exception as exc:  # vLLM missing or not importable with this torch
        print(json.dumps(unavailable(f"{type(exc).__name__}: {exc}")))
        return 0
    import reference_arm

    from prism_infer_b200.models.architecture import Qwen3VLArch

    arch = Qwen3VLArch.qwen3_vl_8b()
    ckpt = args.checkpoint or os.path.join(tempfile.gettempdir(), "prism_ref_qwen3vl8b_random")
    if not args.checkpoint:
        reference_arm.write_checkpoint(ckpt, arch)
    try:
        llm = vllm.LLM(model=ckpt, tensor_parallel_size=args.tp, max_model_len=args.max_model_len, kv_cache_dtype=args.kv_cache_dtype,
                       gpu_memory_utilization=args.gpu_memory_utilization, enforce_eager=args.enforce_eager, enable_prefix_caching=False,
                       limit_mm_per_prompt={"image": max(1, args.images)}, max_num_seqs=max(1, args.batch), dtype="bfloat16",
                       skip_tokenizer_init=False, seed=0)
    except Exception as exc:
        print(json.dumps(unavailable(f"vLLM could not load the checkpoint: {type(exc).__name__}: {exc}")))
        return 0
    rng = np.random.default_rng(0)

    def generate(prompts, max_tokens):
        sp = vllm.SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True, detokenize=False)
        return [list(o.outputs[0].token_ids) for o in llm.generate(prompts, sp, use_tqdm=False)]

    res = measure(generate, lambda: make_requests(arch, rng, batch=args.batch, images=args.images, size=args.size,
                                                  question_tokens=args.question_tokens),
                  output_tokens=args.output_tokens, warmup=args.warmup, repeats=args.repeats)
    record = {"engine": "vllm", "engine_version": getattr(vllm, "__version__", "unknown"), "metric": "qwen3_vl_8b_decode_tpot_ms",
              "value": res["tpot_ms"], "unit": "ms/token", "ttft_ms": res["ttft_ms"], "n_gpus": args.tp, "dtype": "bf16",
              "data": "synthetic (uniform-random images and token ids, random-init weights)",
              "config": {"model": "Qwen3-VL-8B (random init)", "global_batch": args.batch, "images": f"{args.images}x{args.size}x{args.size}",
                         "question_tokens": args.question_tokens, "output_tokens": args.output_tokens, "kv_cache_dtype": args.kv_cache_dtype,
                         "parallelism": f"tp{args.tp}", "enforce_eager": args.enforce_eager,
                         "timing": "(t(K+1 tokens) - t(1 token)) / K through LLM.generate, medians of the repeats"},
              "details": res}
    print(json.dumps(record), flush=True)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as fh:
            json.dump(record, fh, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
