"""Micro-benchmark of the prefill / vision attention kernels (CUDA events, L2 flushed before
every launch): causal GQA attention over fresh bf16 K/V rows, the same over scaled-FP8 pages,
and the bidirectional per-image attention of the vision tower (16 heads x 72).  The library
column is ``torch.nn.functional.scaled_dot_product_attention`` on the same problem.

    python benchmarks/bench_prefill_attention.py [--iters 20]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import ops  # noqa: E402


def timeit(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, device=dev).to(torch.bfloat16)

    for T in (1616, 4096):
        Hq, Hkv, D, page = 32, 8, 128, 256
        qkv = rnd(T, (Hq + 2 * Hkv) * D)
        heads = qkv.view(T, Hq + 2 * Hkv, D)
        q = heads[:, :Hq].contiguous()
        k, v = heads[:, Hq:Hq + Hkv], heads[:, Hq + Hkv:]
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        flops = 4.0 * T * T * D * Hq / 2
        ms = timeit(lambda: ops.varlen_attention(q, k, v, cu, T, causal=True), args.iters, flush)
        qs, ks, vs = (t.transpose(0, 1).unsqueeze(0) for t in (q, k.repeat_interleave(4, 1), v.repeat_interleave(4, 1)))
        lib = timeit(lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True), args.iters, flush)
        print(json.dumps({"case": f"text causal bf16 rows T={T}", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                          "library_ms": round(lib, 4)}), flush=True)
        nblk = (T + page - 1) // page
        cache = ops.KVCache(1, nblk, Hkv, page, D, ops.KV_FP8_SCALED, dev)
        slots = torch.arange(T, dtype=torch.int64, device=dev)
        ops.store_kv(k.contiguous(), v.contiguous(), slots, cache, 0)
        bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(1, -1)
        kvl = torch.tensor([T], dtype=torch.int32, device=dev)
        ms = timeit(lambda: ops.paged_prefill_attention(q, cache, 0, cu, kvl, bt, T), args.iters, flush)
        print(json.dumps({"case": f"text causal scaled-FP8 pages T={T}, page-reading mma.sync kernel", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}), flush=True)
        kw = dict(cu_seqlens_kv=cu, total_kv=T, max_kv_len=T)
        ms = timeit(lambda: ops.paged_prefill_attention(q, cache, 0, cu, kvl, bt, T, **kw), args.iters, flush)
        print(json.dumps({"case": f"text causal scaled-FP8 pages T={T}, gather + tcgen05 kernel", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}), flush=True)
    # a 2048-token chunk over a 14336-token history (chunked prefill of a long video), scaled-FP8 pages
    Hq, Hkv, D, page, Tq, hist = 32, 8, 128, 256, 2048, 14336
    Tk = hist + Tq
    q = rnd(Tq, Hq, D)
    nblk = Tk // page
    cache = ops.KVCache(1, nblk, Hkv, page, D, ops.KV_FP8_SCALED, dev)
    for lo in range(0, Tk, 4096):
        n = min(4096, Tk - lo)
        ops.store_kv(rnd(n, Hkv, D), rnd(n, Hkv, D), torch.arange(lo, lo + n, dtype=torch.int64, device=dev), cache, 0)
    bt = torch.arange(nblk, dtype=torch.int32, device=dev).view(1, -1)
    cu = torch.tensor([0, Tq], dtype=torch.int32, device=dev)
    cu_kv = torch.tensor([0, Tk], dtype=torch.int32, device=dev)
    kvl = torch.tensor([Tk], dtype=torch.int32, device=dev)
    flops = 4.0 * D * Hq * (Tq * hist + Tq * Tq / 2)
    for name, kw in (("page-reading mma.sync kernel", {}), ("gather + tcgen05 kernel", dict(cu_seqlens_kv=cu_kv, total_kv=Tk, max_kv_len=Tk))):
        ms = timeit(lambda: ops.paged_prefill_attention(q, cache, 0, cu, kvl, bt, Tq, **kw), args.iters, flush)
        print(json.dumps({"case": f"chunk {Tq} over history {hist}, scaled-FP8 pages, {name}", "ms": round(ms, 4),
                          "tflops": round(flops / ms / 1e9, 1)}), flush=True)
    n_img, seg, H, hd = 8, 784, 16, 72
    N = n_img * seg
    qkv = rnd(N, 3 * H * hd)
    hv = qkv.view(N, 3, H, hd)
    cu = torch.arange(0, N + 1, seg, dtype=torch.int32, device=dev)
    flops = 4.0 * n_img * seg * seg * hd * H
    ms = timeit(lambda: ops.varlen_attention(hv[:, 0], hv[:, 1], hv[:, 2], cu, seg, causal=False), args.iters, flush)
    qs, ks, vs = (hv[:, i].reshape(n_img, seg, H, hd).transpose(1, 2) for i in range(3))
    lib = timeit(lambda: F.scaled_dot_product_attention(qs, ks, vs), args.iters, flush)
    print(json.dumps({"case": f"vision {n_img} x {seg} patches, 16 heads x 72", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                      "library_ms": round(lib, 4)}), flush=True)


if __name__ == "__main__":
    main()
