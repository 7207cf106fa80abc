"""Step timeline of the persistent decode kernel (``ops/csrc/decode_layers.cu``).

Worker thread 0 of every CTA stores the GPU-wide nanosecond timer at each step boundary of each layer; this
script runs a few decode steps of a random-init model with the recording on and prints, per
step of a layer, the mean and the maximum over CTAs (averaged over layers) in microseconds, next
to the device time of a whole decode step with the recording off.  Most rows are waits for other
CTAs' values (the kernel has no barriers: a CTA proceeds as soon as the words it polls carry the
hand-off's sequence number), so a long row names the hand-off the layer is bound by.

    python benchmarks/profile_decode_layers.py [--model random:qwen3-vl-8b] [--context 1616] [--batch 1]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

PHASES = (
    "poll residual*w + 1/rms into shared memory (QKV input)",
    "QKV epilogue (waits for the CTA's MMAs)",
    "attention: q/k/v rows from the QKV words, KV store",
    "attention: fold staged cached tokens",
    "attention: merge warps, publish the split",
    "attention: split 0 merges the splits",
    "poll attention output into shared memory (o_proj input)",
    "o_proj epilogue",
    "residual tile owner: sum o_proj words, publish residual*w",
    "poll residual*w + 1/rms (gate/up input)",
    "gate/up epilogue",
    "activation tile owner: SwiGLU",
    "poll activations (down input)",
    "down epilogue",
    "residual tile owner: sum down words, publish residual*w",
)


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
    tl = plan.timeline.cpu().double()  # [grid, layers, 16]
    plan.record_timeline(False)
    ops.native.check_status()
    # stamps are nanoseconds of the GPU-wide timer: one time axis for all CTAs
    layers = slice(1, None) if tl.shape[1] > 1 else slice(0, None)
    tl = tl[:, layers] / 1000.0
    d = tl[:, :, 1:] - tl[:, :, :-1]  # microseconds per step of a layer
    mean = d.mean(dim=(0, 1))
    worst = d.max(dim=0).values.mean(dim=0)
    layer_us = float((tl[:, :, -1] - tl[:, :, 0]).mean())
    rows = [{"phase": name, "mean_us": round(float(m), 2), "max_over_ctas_us": round(float(w), 2)} for name, m, w in zip(PHASES, mean, worst)]
    print(f"model {args.model}  batch {B}  context {n}  grid {plan.grid}  slabs {plan.slabs}  ring stages {plan.stages}  "
          f"activation slots {plan.xslots}")
    print(f"step (layers + embedding + final norm), recording off: {plain_ms:.3f} ms; one layer on the timeline: {layer_us:.1f} us")
    print("time spent in each step of a layer (per CTA):")
    for r in rows:
        print(f"  {r['phase']:<58s} mean {r['mean_us']:8.2f} us   max over CTAs {r['max_over_ctas_us']:8.2f} us")
    # when each step ENDS on the layer's own time axis (0 = the first CTA entering the layer): first, mean and last CTA
    rel = tl - tl[:, :, 0].min(dim=0).values[None, :, None]
    print("end of each step since the first CTA entered the layer (first / mean / last CTA):")
    ends = []
    for k, name in enumerate(("enter the layer",) + PHASES):
        col = rel[:, :, k]
        lo, mid, hi = float(col.min(dim=0).values.mean()), float(col.mean()), float(col.max(dim=0).values.mean())
        ends.append({"step": name, "first_us": round(lo, 2), "mean_us": round(mid, 2), "last_us": round(hi, 2)})
        print(f"  {name:<58s} {lo:8.2f} {mid:8.2f} {hi:8.2f}")
    if args.json:
        with open(args.json, "w") as fh:
            json.dump({"model": args.model, "batch": B, "context": n, "step_ms": plain_ms, "layer_us": layer_us, "phases": rows, "ends": ends}, fh, indent=1)


if __name__ == "__main__":
    main()
