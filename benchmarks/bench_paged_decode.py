"""Kernel micro-benchmark with a correctness gate: paged decode attention over bf16, FP8 and scaled-FP8 pages against a
dequantise-then-softmax statement of the same computation written here in plain PyTorch, over a sweep of batch sizes,
context lengths and page sizes.  Reports the time per call, the achieved KV bandwidth and its fraction of the measured
copy peak, and the largest / mean absolute difference to the statement; a case whose difference exceeds the gates makes
the run fail.  Mirrors the reference's ``benchmarks/bench_paged_decode.py``.

    python benchmarks/bench_paged_decode.py [--batch-sizes 1,8,32,128] [--context-lens 2048] [--page-sizes 256]
        [--cache-dtypes scaled_fp8,bf16] [--num-heads 32 --num-kv-heads 8 --head-dim 128] [--output rec.json]

``--device cpu`` runs the CPU statements of the ops (no bandwidth claim: a check that the script and the gates work).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from prism_infer_b200 import ops  # noqa: E402

CACHE_MODES = {"bf16": ops.KV_BF16, "fp8": ops.KV_FP8, "scaled_fp8": ops.KV_FP8_SCALED}


def ints(text: str) -> list[int]:
    values = [int(x) for x in str(text).split(",") if x.strip()]
    if not values or any(v <= 0 for v in values):
        raise argparse.ArgumentTypeError(f"expected positive integers separated by commas, got {text!r}")
    return values


def fill_cache(cache, mode: int, seed: int) -> None:
    g = torch.Generator(device="cpu").manual_seed(seed)
    shape = tuple(cache.payload.shape)
    if mode == ops.KV_BF16:
        cache.payload.copy_(torch.randn(shape, generator=g).to(cache.payload.dtype))
        return
    raw = torch.randint(0, 120, shape, generator=g, dtype=torch.uint8)           # E4M3 bytes of finite, positive values
    sign = torch.randint(0, 2, shape, generator=g, dtype=torch.uint8) * 128
    cache.payload.view(torch.uint8).copy_((raw | sign).to(cache.payload.device))
    if cache.scales is not None:
        cache.scales.copy_(torch.empty(tuple(cache.scales.shape)).uniform_(0.005, 0.02, generator=g))


def statement(q: torch.Tensor, cache, block_tables: torch.Tensor, context_lens: torch.Tensor) -> torch.Tensor:
    """Gather every sequence's pages, dequantise, repeat the KV heads over their query group, softmax in fp32."""
    B, Hq, D = q.shape
    Hkv, page = cache.num_kv_heads, cache.page
    k_all = cache.k(0).float()
    v_all = cache.v(0).float()
    if cache.scales is not None:
        k_all = k_all * cache.k_scale(0).float().unsqueeze(-1)
        v_all = v_all * cache.v_scale(0).float().unsqueeze(-1)
    out = torch.empty((B, Hq, D), dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(context_lens[b])
        pages = block_tables[b, : -(-n // page)].long()
        k = k_all[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]           # [Hkv, n, D]
        v = v_all[pages].permute(1, 0, 2, 3).reshape(Hkv, -1, D)[:, :n]
        k = k.repeat_interleave(Hq // Hkv, dim=0)
        v = v.repeat_interleave(Hq // Hkv, dim=0)
        s = torch.einsum("hd,hnd->hn", q[b].float(), k) * D ** -0.5
        out[b] = torch.einsum("hn,hnd->hd", torch.softmax(s, dim=-1), v)
    return out


def run_case(*, device: torch.device, mode_name: str, batch: int, ctx: int, page: int, heads: int, kv_heads: int, head_dim: int,
             warmup: int, repeat: int, seed: int, flush: torch.Tensor | None) -> dict:
    mode = CACHE_MODES[mode_name]
    per_seq = -(-ctx // page)
    n_pages = batch * per_seq
    kw = {} if device.type == "cuda" else {"dtype": torch.float32}
    cache = ops.KVCache(1, n_pages, kv_heads, page, head_dim, mode, device, **kw)
    fill_cache(cache, mode, seed)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed + 1)).to(torch.int32)
    bt = perm.view(batch, per_seq).to(device)                                     # pages scattered over the pool
    lens = torch.full((batch,), ctx, dtype=torch.int32, device=device)
    q = torch.randn(batch, heads, head_dim, generator=torch.Generator().manual_seed(seed + 2))
    q = q.to(device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    out = torch.empty_like(q)
    for _ in range(warmup):
        ops.paged_decode_attention(q, cache, 0, bt, lens, out=out)
    total = 0.0
    for _ in range(repeat):
        if device.type == "cuda":
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            ops.paged_decode_attention(q, cache, 0, bt, lens, out=out)
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        else:
            t0 = time.perf_counter()
            ops.paged_decode_attention(q, cache, 0, bt, lens, out=out)
            total += (time.perf_counter() - t0) * 1e3
    ms = total / repeat
    diff = (out.float() - statement(q, cache, bt, lens)).abs()
    kv_bytes = 2 * batch * ctx * kv_heads * head_dim * cache.payload.element_size() + (2 * batch * ctx * kv_heads * 4 if cache.scales is not None else 0)
    return {"cache_dtype": mode_name, "batch": batch, "context_len": ctx, "page_size": page, "num_heads": heads, "num_kv_heads": kv_heads,
            "head_dim": head_dim, "ms": ms, "kv_bytes": kv_bytes, "kv_gbs": kv_bytes / ms / 1e6,
            "max_abs_diff": float(diff.max()), "mean_abs_diff": float(diff.mean())}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch-sizes", "--batches", type=ints, default=[1, 8, 32, 128])
    ap.add_argument("--context-lens", "--ctx", type=ints, default=[2048])
    ap.add_argument("--page-sizes", type=ints, default=[256])
    ap.add_argument("--cache-dtypes", default="scaled_fp8,bf16", help=f"comma-separated, of {sorted(CACHE_MODES)}")
    ap.add_argument("--num-heads", type=int, default=32)
    ap.add_argument("--num-kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", "--iters", type=int, default=20)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--max-abs-diff", type=float, default=2e-2, help="gate on the largest difference to the statement")
    ap.add_argument("--mean-abs-diff", type=float, default=2e-3)
    ap.add_argument("--output", default="")
    ap.add_argument("--overwrite", action="store_true")
    args = ap.parse_args(argv)
    dtypes = [d.strip() for d in args.cache_dtypes.split(",") if d.strip()]
    for d in dtypes:
        if d not in CACHE_MODES:
            ap.error(f"unknown cache dtype {d!r}; known: {sorted(CACHE_MODES)}")
    if args.num_heads % args.num_kv_heads:
        ap.error("--num-heads must be a multiple of --num-kv-heads")
    if args.output and os.path.exists(args.output) and not args.overwrite:
        ap.error(f"{args.output} exists; pass --overwrite to replace it")
    device = torch.device(args.device)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm = json.load(open(peaks_path))["hbm_gbs"] if os.path.exists(peaks_path) else 6650.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if device.type == "cuda" else None
    rows, failed = [], []
    for name in dtypes:
        for page in args.page_sizes:
            for ctx in args.context_lens:
                for batch in args.batch_sizes:
                    row = run_case(device=device, mode_name=name, batch=batch, ctx=ctx, page=page, heads=args.num_heads,
                                   kv_heads=args.num_kv_heads, head_dim=args.head_dim, warmup=args.warmup, repeat=args.repeat,
                                   seed=args.seed, flush=flush)
                    row["passed"] = row["max_abs_diff"] <= args.max_abs_diff and row["mean_abs_diff"] <= args.mean_abs_diff
                    if device.type == "cuda":
                        row["frac_hbm_of_measured"] = row["kv_gbs"] / hbm
                    rows.append(row)
                    if not row["passed"]:
                        failed.append(row)
                    print(json.dumps({k: (round(v, 5) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
    record = {"record_type": "paged_decode_microbenchmark", "device": str(device), "gates": {"max_abs_diff": args.max_abs_diff,
              "mean_abs_diff": args.mean_abs_diff}, "hbm_gbs_measured_peak": hbm if device.type == "cuda" else None,
              "timing": "CUDA events, L2 flushed before every call" if device.type == "cuda" else "host clock", "rows": rows,
              "passed": not failed}
    if args.output:
        with open(args.output, "w", encoding="utf-8") as fh:
            json.dump(record, fh, indent=1)
    if failed:
        print(f"{len(failed)} case(s) exceed the difference gates", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
