"""Phase timeline of the persistent decode kernel (``ops/csrc/decode_layers.cu``).

Worker thread 0 of every CTA stores its SM clock at each phase boundary of each layer; this
script runs a few decode steps of a random-init model with the recording on and prints, per
phase, the mean and the maximum over CTAs (averaged over layers) in microseconds, next to the
device time of a step with the recording off.  The barrier rows are waits: a long barrier after a
short phase means some other CTA's phase was long.

    python benchmarks/profile_decode_layers.py [--model random:qwen3-vl-8b] [--context 1616] [--batch 1]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

PHASES = ("embedding rows -> residual, xw (first layer only)", "barrier (first layer only)", "qkv epilogue (waits for the GEMM)",
          "barrier", "q/k/v rows + attention", "barrier", "o_proj epilogue + reduce tails", "barrier",
          "gate/up epilogue + swiglu tails", "barrier", "down epilogue + reduce tails", "barrier")
N_PHASE_STAMPS = 13


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--context", type=int, default=1616)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    from prism_infer_b200 import ops
    from prism_infer_b200.config import resolve_arch
    from prism_infer_b200.models.qwen3_vl import AttnMeta, Qwen3VLModel
    from prism_infer_b200.models.weights import iter_random_weights

    arch = resolve_arch(args.model)
    t = arch.text
    model = Qwen3VLModel(arch, device="cuda", dtype=torch.bfloat16, load_vision=False)
    model.load(iter_random_weights(arch, dtype=torch.bfloat16, device="cuda", seed=0), strict=False)
    page = 256
    B, n = args.batch, args.context
    pages = -(-(n + args.steps + 2) // page)
    cache = ops.KVCache(t.num_layers, B * pages + 1, t.num_kv_heads, page, t.head_dim, ops.KV_FP8_SCALED, "cuda")
    cache.payload.view(torch.uint8).random_(0, 120)  # any finite E4M3 codes: timing does not depend on the values
    cache.scales.fill_(0.01)
    bt = torch.arange(B * pages, dtype=torch.int32).view(B, pages).cuda()
    ids = torch.randint(0, t.vocab_size, (B,), device="cuda")
    pos = torch.full((3, B), n, dtype=torch.int32, device="cuda")
    slots = (bt[:, n // page].long() * page + n % page).contiguous()
    ctx = torch.full((B,), n + 1, dtype=torch.int32, device="cuda")
    meta = AttnMeta(is_prefill=False, block_tables=bt, slots=slots, context_lens=ctx)
    plan = model._decode_plan(cache, B)
    assert plan is not None, "the persistent decode kernel does not apply to this model shape"

    def timed(k: int) -> float:
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(k):
            model.forward(ids, pos, meta, cache)
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / k

    timed(3)
    plain_ms = timed(args.steps)
    plan.record_timeline(True)
    timed(2)
    tl = plan.timeline.cpu().double()  # [grid, layers, 20]
    plan.record_timeline(False)
    ops.native.check_status()
    try:
        mhz = float(torch.cuda.clock_rate())  # current SM clock
    except Exception:  # no NVML binding: the part's maximum
        mhz = 1965.0
    sub = tl[:, :, N_PHASE_STAMPS:]
    tl = tl[:, :, :N_PHASE_STAMPS]
    d = (tl[:, :, 1:] - tl[:, :, :-1]) / mhz  # microseconds per phase
    layers = slice(1, None) if d.shape[1] > 1 else slice(0, None)
    mean = d[:, layers].mean(dim=(0, 1))
    worst = d[:, layers].max(dim=0).values.mean(dim=0)
    layer_us = float((tl[:, layers, -1] - tl[:, layers, 0]).mean() / mhz)
    rows = [{"phase": name, "mean_us": round(float(m), 2), "max_over_ctas_us": round(float(w), 2)} for name, m, w in zip(PHASES, mean, worst)]
    print(f"model {args.model}  batch {B}  context {n}  grid {plan.grid}  slabs {plan.slabs}  stages {plan.stages}  sm clock {mhz} MHz")
    print(f"step (layers + embedding + final norm), recording off: {plain_ms:.3f} ms; one layer on the timeline: {layer_us:.1f} us")
    for r in rows:
        print(f"  {r['phase']:<40s} mean {r['mean_us']:8.2f} us   max over CTAs {r['max_over_ctas_us']:8.2f} us")
    # inside the attention item (CTAs that had one): entry, rows built, CTA barrier, tokens folded, warps merged,
    # partials published + arrival counted, end
    names = ("build q/k/v rows (slab sums, norm, rotary, KV store)", "CTA barrier", "fold cached tokens", "merge warps",
             "publish partials, fence, arrival counter", "last split: merge all splits (others: nothing)")
    has = (sub[:, layers, 0] > 0) & (sub[:, layers, 6] > 0)
    if bool(has.any()):
        dd = (sub[:, layers, 1:] - sub[:, layers, :-1]) / mhz
        print("  inside one attention item:")
        for k, name in enumerate(names):
            vals = dd[..., k][has]
            print(f"    {name:<60s} mean {float(vals.mean()):7.2f} us   max {float(vals.max()):7.2f} us")
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"model": args.model, "batch": B, "context": n, "step_ms": plain_ms, "layer_us": layer_us, "phases": rows}, fh, indent=1)


if __name__ == "__main__":
    main()
