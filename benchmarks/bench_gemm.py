"""Micro-benchmark of the tcgen05 GEMM family against cuBLAS (``torch.matmul``).

Decode-shaped (weight-streaming, few tokens) cases report achieved HBM bandwidth, prefill-
shaped cases report TFLOP/s; both as a fraction of the measured peaks in
``MEASURED_PEAKS.json`` when that file exists.  Timing: CUDA events on the launching stream,
warm-up, an L2 flush (a 256 MB write) before every timed launch.

    python benchmarks/bench_gemm.py [--iters 20] [--json out.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import ops  # noqa: E402


def peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return json.load(fh)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


def timeit(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    return total / iters  # ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="", help="substring filter on case names")
    args = ap.parse_args()
    pk = peaks()
    dev = torch.device("cuda:0")
    ops.apply_tuning()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []
    cases = [
        # name, T, M, K, kind
        ("qkv b1", 1, 6144, 4096, "plain"), ("o b1", 1, 4096, 4096, "plain"), ("gate_up b1", 1, 24576, 4096, "plain"),
        ("down b1", 1, 4096, 12288, "plain"), ("lm_head b1", 1, 151936, 4096, "plain"),
        ("gate_up dual b1", 1, 12288, 4096, "dual"), ("gate_up dual b32", 32, 12288, 4096, "dual"),
        ("qkv b128", 128, 6144, 4096, "plain"), ("down b128", 128, 4096, 12288, "plain"),
        ("qkv t2048", 2048, 6144, 4096, "plain"), ("down t2048", 2048, 4096, 12288, "plain"),
        ("gate_up dual t2048", 2048, 12288, 4096, "dual"), ("o t8192", 8192, 4096, 4096, "plain"),
        ("vit fc1 t6272", 6272, 4304, 1152, "plain"), ("vit qkv t6272", 6272, 3456, 1152, "plain"),
        ("vit proj t6272", 6272, 1152, 1152, "plain"), ("vit fc2 t6272", 6272, 1152, 4304, "plain"),
        ("qkv t1616", 1616, 6144, 4096, "plain"), ("gate_up dual t1616", 1616, 12288, 4096, "dual"),
    ]
    for name, T, M, K, kind in cases:
        if args.only and args.only not in name:
            continue
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        rowsW = 2 * M if kind == "dual" else M
        w = (torch.randn(rowsW, K, device=dev) * K ** -0.5).to(torch.bfloat16)
        best = None
        if kind == "dual":
            variants = {"dual": lambda: ops.gate_up_swiglu(x, w, bn=16 if T <= 16 else 0)}
            ref = lambda: torch.nn.functional.silu((x @ w.t())[:, :M]) * (x @ w.t())[:, M:]  # noqa: E731
        elif T <= 128:
            variants = {}
            for s in sorted({1, ops.choose_splits(M, K, T), 2, 4, 8}):
                out = torch.empty((ops.effective_splits(K, s), T, M), dtype=torch.float32, device=dev)
                variants[f"split{s}"] = (lambda s=s, out=out: ops.linear_partial(x, w, s, out, bn=16 if T <= 16 else 0))
            ref = lambda: x @ w.t()  # noqa: E731
        else:
            out = torch.empty((T, M), dtype=torch.bfloat16, device=dev)
            variants = {"bn256": lambda: ops.linear(x, w, out=out, bn=256), "bn128": lambda: ops.linear(x, w, out=out, bn=128),
                        "persistent": lambda: ops.linear(x, w, out=out)}
            ref = lambda: x @ w.t()  # noqa: E731
        t_ref = timeit(ref, args.iters, flush)
        all_ms = {}
        for vname, fn in variants.items():
            ms = timeit(fn, args.iters, flush)
            all_ms[vname] = round(ms, 5)
            if best is None or ms < best[1]:
                best = (vname, ms)
        ms = best[1]
        bytes_ = rowsW * K * 2 + T * K * 2 + T * M * 2
        flops = 2.0 * T * rowsW * K
        row = {
            "case": name, "T": T, "M": rowsW, "K": K, "variant": best[0], "ms": round(ms, 5), "all_ms": all_ms, "cublas_ms": round(t_ref, 5),
            "gbs": round(bytes_ / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1),
            "frac_hbm_of_measured": round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3),
            "frac_bf16_of_measured": round(flops / ms / 1e9 / pk["bf16_tflops"], 3),
        }
        rows.append(row)
        print(json.dumps(row), flush=True)
    # epilogue forms of the vision tower on the persistent kernel
    for name, T, M, K, form in (("vit proj", 6272, 1152, 1152, "bias+residual in place"), ("vit fc2", 6272, 1152, 4304, "bias+residual in place"),
                                ("vit fc1", 6272, 4304, 1152, "bias+gelu_tanh"), ("vit proj", 6272, 1152, 1152, "bias+residual separate")):
        if args.only and args.only not in f"{name} epilogue":
            continue
        x = torch.randn(T, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(M, K, device=dev) * K ** -0.5).to(torch.bfloat16)
        b = torch.randn(M, device=dev).to(torch.bfloat16)
        res = torch.randn(T, M, device=dev).to(torch.bfloat16)
        out = torch.empty_like(res)
        if form == "bias+residual in place":
            fn = lambda: ops.linear(x, w, bias=b, residual=res, out=res)  # noqa: E731
        elif form == "bias+residual separate":
            fn = lambda: ops.linear(x, w, bias=b, residual=res, out=out)  # noqa: E731
        else:
            fn = lambda: ops.linear(x, w, bias=b, act="gelu_tanh", out=out)  # noqa: E731
        plain = timeit(lambda: ops.linear(x, w, out=out), args.iters, flush)
        ms = timeit(fn, args.iters, flush)
        row = {"case": f"{name} epilogue {form}", "T": T, "M": M, "K": K, "ms": round(ms, 5), "plain_ms": round(plain, 5)}
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"peaks": pk, "rows": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
