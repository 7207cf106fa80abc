"""Kernel micro-benchmark: paged decode attention (scaled-FP8 and bf16 pages) against the
dequantise-then-SDPA statement of the same computation, achieved HBM bandwidth as a fraction
of the measured copy peak.  Mirrors the reference's ``benchmarks/bench_paged_decode.py``.

    python benchmarks/bench_paged_decode.py [--ctx 2048] [--batches 1,8,32,128]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import ops  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--batches", default="1,8,32,128")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm = json.load(open(peaks_path))["hbm_gbs"] if os.path.exists(peaks_path) else 6650.0
    dev = torch.device("cuda:0")
    Hq, Hkv, D, page = 32, 8, 128, 256
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for mode, name in ((ops.KV_FP8_SCALED, "scaled_fp8"), (ops.KV_BF16, "bf16")):
        for B in [int(b) for b in args.batches.split(",")]:
            n_pages = B * (-(-args.ctx // page))
            cache = ops.KVCache(1, n_pages, Hkv, page, D, mode, dev)
            if mode == ops.KV_BF16:
                cache.payload.normal_()
            else:
                cache.payload.view(torch.uint8).random_(0, 120)
                cache.scales.uniform_(0.005, 0.02)
            bt = torch.arange(n_pages, dtype=torch.int32, device=dev).view(B, -1)
            ctx = torch.full((B,), args.ctx, dtype=torch.int32, device=dev)
            q = torch.randn(B, Hq, D, device=dev).to(torch.bfloat16)
            out = torch.empty_like(q)
            for _ in range(3):
                ops.paged_decode_attention(q, cache, 0, bt, ctx, out=out)
            total = 0.0
            for _ in range(args.iters):
                flush.zero_()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                ops.paged_decode_attention(q, cache, 0, bt, ctx, out=out)
                e.record()
                torch.cuda.synchronize()
                total += s.elapsed_time(e)
            ms = total / args.iters
            bytes_ = 2 * B * args.ctx * Hkv * D * cache.payload.element_size() + (2 * B * args.ctx * Hkv * 4 if cache.scales is not None else 0)
            print(json.dumps({"kv": name, "batch": B, "ctx": args.ctx, "ms": round(ms, 4), "gbs": round(bytes_ / ms / 1e6, 1),
                              "frac_hbm_of_measured": round(bytes_ / ms / 1e6 / hbm, 3)}), flush=True)


if __name__ == "__main__":
    main()
