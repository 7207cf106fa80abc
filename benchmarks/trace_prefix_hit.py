"""One cold multimodal request followed by a same-media, different-question request, traced
(reference ``benchmarks/trace_working_set_prefix.py``, ``benchmarks/audit_working_set_prefix_trace.py``).

Engine construction and one warm-up request on other media stay outside the traced span.  The
span is bracketed by ``cudaProfilerStart`` / ``cudaProfilerStop``, so the same command can run
under ``nsys profile --capture-range=cudaProfilerApi`` (or ``ncu --profile-from-start off``);
inside it the two requests run under the marker regions ``cold_request`` and
``prefix_hit_request`` of a ``performance_profile`` session, which also pushes them as NVTX
ranges ``prism::cold_request`` / ``prism::prefix_hit_request``.

The record holds the counter evidence (the second request probed, hit, ran no vision patches and
reported cached tokens), the audit of the regions nested in each marker (vision ranges in the
cold request, none in the hit) and both requests' time to first token.  Anything unexpected
raises.  With ``--sqlite`` an Nsight Systems export of an earlier traced run is audited instead
(nothing is executed).

    python benchmarks/trace_prefix_hit.py [--images 8] [--size 448] [--mode visual_compact_scaled_fp8] --out trace.json
    python benchmarks/trace_prefix_hit.py --sqlite capture.sqlite --evidence trace.json --out audit.json
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Any, Sequence

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import LLM, SamplingParams  # noqa: E402
from prism_infer_b200.analysis import prefix_trace as pt  # noqa: E402
from prism_infer_b200.analysis.performance_profile import performance_profile  # noqa: E402
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs  # noqa: E402
from prism_infer_b200.observability import profile_region  # noqa: E402


def _one_request(llm, inputs, sp) -> dict[str, Any]:
    """Run one prepared request to completion -> its metric record, first-token time and the
    vision patches its batches ran."""
    n_req = len(llm.metrics_snapshot()["engine"]["requests"])
    n_batch = len(llm.metrics_snapshot()["engine"]["batches"])
    t0 = time.perf_counter()
    rid = llm.add_prepared_image_request(inputs, sp)
    first_ms = None
    tokens: list[int] = []
    while not llm.is_finished():
        res = llm.step_result()
        if first_ms is None and any(o.request_id == rid for o in res.outputs):
            first_ms = (time.perf_counter() - t0) * 1e3
        for o in res.finished:
            if o.request_id == rid:
                tokens = list(o.token_ids)
    snap = llm.metrics_snapshot()["engine"]
    (metric,) = [r for r in snap["requests"][n_req:] if r["request_id"] == rid]
    patches = sum(int(b.get("vision_patches", 0)) for b in snap["batches"][n_batch:])
    return {"metric": metric, "first_token_wall_ms": first_ms, "vision_patches": patches, "token_ids": tokens}


def run_prefix_trace(llm, images: Sequence[np.ndarray], warm_images: Sequence[np.ndarray], question_a: Sequence[int],
                     question_b: Sequence[int], sp: SamplingParams, *, cuda_profiler_range: bool = True) -> dict[str, Any]:
    import torch

    if list(question_a) == list(question_b):
        raise ValueError("the two requests must ask different questions")
    proc = PatchProcessor(llm.arch)
    cold_in = prepare_image_inputs(proc, llm.tokenizer, list(question_a), list(images))
    hit_in = prepare_image_inputs(proc, llm.tokenizer, list(question_b), list(images))
    _one_request(llm, prepare_image_inputs(proc, llm.tokenizer, list(question_a), list(warm_images)), sp)  # untraced warm-up
    cuda = torch.cuda.is_available()
    counters = lambda: {k: int(v) for k, v in llm.multimodal_prefix_cache_metadata().items() if k in pt.PREFIX_COUNTERS}  # noqa: E731
    before = counters()
    if cuda and cuda_profiler_range:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        with performance_profile({"tool": "trace_prefix_hit"}) as session:
            with profile_region(pt.COLD_MARKER, cuda=True):
                cold = _one_request(llm, cold_in, sp)
            after_cold = counters()
            with profile_region(pt.HIT_MARKER, cuda=True):
                hit = _one_request(llm, hit_in, sp)
            after_hit = counters()
            record = session.finalize()
    finally:
        if cuda and cuda_profiler_range:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
    evidence = pt.validate_prefix_hit_evidence(before, after_cold, after_hit, cold["metric"], hit["metric"],
                                               cold_vision_patches=cold["vision_patches"], hit_vision_patches=hit["vision_patches"])
    audit = pt.audit_prefix_trace(pt.nested_names_from_profile(record, pt.COLD_MARKER),
                                  pt.nested_names_from_profile(record, pt.HIT_MARKER), evidence)
    if not audit["passed"]:
        raise RuntimeError(json.dumps(audit, sort_keys=True))
    markers = {r["name"]: r for r in record["regions"] if r["name"] in (pt.COLD_MARKER, pt.HIT_MARKER)}
    return {
        "record_type": "prefix_hit_trace", "evidence": evidence, "audit": audit,
        "cold_request": {"first_token_wall_ms": cold["first_token_wall_ms"], "ttft_ms": cold["metric"].get("ttft_ms"),
                         "span_cpu_ms": markers[pt.COLD_MARKER]["cpu_ms"], "span_cuda_ms": markers[pt.COLD_MARKER].get("cuda_ms"),
                         "prompt_tokens": cold["metric"]["prompt_tokens"]},
        "prefix_hit_request": {"first_token_wall_ms": hit["first_token_wall_ms"], "ttft_ms": hit["metric"].get("ttft_ms"),
                               "span_cpu_ms": markers[pt.HIT_MARKER]["cpu_ms"], "span_cuda_ms": markers[pt.HIT_MARKER].get("cuda_ms"),
                               "prompt_tokens": hit["metric"]["prompt_tokens"]},
        "region_totals": record["totals"],
    }


def audit_nsys_export(sqlite_path: str | Path, evidence_record: dict[str, Any]) -> dict[str, Any]:
    from prism_infer_b200.analysis.nsys_trace import nvtx_ranges, open_export

    con = open_export(sqlite_path)
    try:
        ranges = nvtx_ranges(con)
    finally:
        con.close()
    audit = pt.audit_prefix_trace(pt.nested_names_from_nvtx(ranges, pt.COLD_MARKER), pt.nested_names_from_nvtx(ranges, pt.HIT_MARKER),
                                  evidence_record["evidence"])
    if not audit["passed"]:
        raise RuntimeError(json.dumps(audit, sort_keys=True))
    return audit


def _write_new(path: str, value: dict[str, Any]) -> None:
    out = Path(path)
    if out.exists():
        raise FileExistsError(f"refusing to overwrite {out}")
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps(value, indent=2, sort_keys=True) + "\n", encoding="utf-8")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="random:qwen3-vl-8b")
    ap.add_argument("--images", type=int, default=8)
    ap.add_argument("--size", type=int, default=448)
    ap.add_argument("--question-tokens", type=int, default=32)
    ap.add_argument("--max-tokens", type=int, default=8)
    ap.add_argument("--mode", default="visual_compact_scaled_fp8")
    ap.add_argument("--device", default=None)
    ap.add_argument("--sqlite", default="", help="audit this Nsight Systems export instead of running")
    ap.add_argument("--evidence", default="", help="record of the traced run that produced --sqlite")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if args.sqlite:
        if not args.evidence:
            ap.error("--sqlite needs --evidence")
        result = audit_nsys_export(args.sqlite, json.loads(Path(args.evidence).read_text(encoding="utf-8")))
    else:
        llm = LLM(args.model, device=args.device, max_model_len=8192, kvcache_block_size=256, num_kvcache_blocks=256,
                  compression_mode=args.mode, max_num_seqs=4, max_num_batched_tokens=16384, max_chunk_size=8192,
                  cpu_kv_cache_ratio=0.0, enable_prefix_caching=True)
        rng = np.random.default_rng(0)
        mk = lambda: [rng.integers(0, 256, (args.size, args.size, 3), dtype=np.uint8) for _ in range(args.images)]  # noqa: E731
        vocab = min(150000, llm.arch.text.vocab_size - 1)
        sp = SamplingParams(temperature=0.0, max_tokens=args.max_tokens, ignore_eos=True)
        try:
            result = run_prefix_trace(llm, mk(), mk(), rng.integers(0, vocab, args.question_tokens).tolist(),
                                      rng.integers(0, vocab, args.question_tokens).tolist(), sp)
        finally:
            llm.exit()
        result["config"] = {"model": args.model, "images": args.images, "size": args.size, "mode": args.mode,
                            "question_tokens": args.question_tokens, "max_tokens": args.max_tokens}
    if args.out:
        _write_new(args.out, result)
    brief = {"passed": result.get("audit", result).get("passed"), "checks": result.get("audit", result).get("checks")}
    for k in ("cold_request", "prefix_hit_request"):
        if k in result:
            brief[k] = result[k]
    print(json.dumps(brief, sort_keys=True))


if __name__ == "__main__":
    main()
