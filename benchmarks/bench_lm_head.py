"""LM head of a greedy decode step at 8B widths (151936 x 4096): the bf16 head (tcgen05 GEMM with fp32 logits +
arg-max) against the E4M3 candidate head with its exact rerank, CUDA events, 256 MB L2 flush before every launch.

    python benchmarks/bench_lm_head.py [--iters 20] [--batches 1,2,4]
"""

from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from prism_infer_b200 import ops  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batches", default="1,2,4")
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--hidden", type=int, default=4096)
    args = ap.parse_args()
    V, H = args.vocab, args.hidden
    w = (torch.randn(V, H, device="cuda") * H ** -0.5).to(torch.bfloat16)
    codes, scale = ops.quantize_lm_head_fp8(w)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn) -> float:
        ts = []
        for _ in range(args.iters + 3):
            flush.zero_()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts = sorted(ts[3:])
        return ts[len(ts) // 2] * 1e3

    for B in (int(b) for b in args.batches.split(",")):
        x = torch.randn(B, H, device="cuda").to(torch.bfloat16)
        t_fp8 = timeit(lambda: ops.lm_head_fp8_greedy(x, codes, scale, w))
        t_bf = timeit(lambda: ops.sample(ops.linear_partial(x, w, 1)[0], None))
        same = bool(torch.equal(ops.lm_head_fp8_greedy(x, codes, scale, w), ops.sample(ops.linear_partial(x, w, 1)[0], None)))
        print(f"batch {B}: E4M3 candidates + rerank {t_fp8:.1f} us ({V * H / t_fp8 / 1e6:.2f} TB/s of E4M3 bytes); "
              f"bf16 head + arg-max {t_bf:.1f} us ({2 * V * H / t_bf / 1e6:.2f} TB/s); same tokens: {same}")


if __name__ == "__main__":
    main()
