"""Latency aggregation for online-serving runs (reference
``prism_infer/analysis/online_serving.py:14-243``): linear-interpolation percentiles at
``(n - 1) * q``, per-request TTFT / end-to-end / TPOT distributions, output tokens per
second over the run duration, and *recomputed prompt tokens* = sum over completed requests
of ``max(0, prompt_tokens - cached_tokens)``."""

from __future__ import annotations

from math import isfinite
from typing import Mapping, Sequence

ONLINE_SUMMARY_SCHEMA_VERSION = 2


def percentile(values: Sequence[float], q: float) -> float:
    if not values:
        raise ValueError("percentile requires non-empty values")
    if not 0.0 <= q <= 1.0:
        raise ValueError("quantile must be in [0, 1]")
    xs = sorted(float(v) for v in values)
    if any(not isfinite(v) for v in xs):
        raise ValueError("percentile values must be finite")
    pos = (len(xs) - 1) * q
    lo = int(pos)
    hi = min(lo + 1, len(xs) - 1)
    w = pos - lo
    return min(xs[hi], xs[lo] + (xs[hi] - xs[lo]) * w)  # exact between equal neighbours, never above the upper one


def summarize_distribution(values: Sequence[float]) -> dict[str, float | int]:
    if not values:
        return {"count": 0, "min": 0.0, "max": 0.0, "mean": 0.0, "p50": 0.0, "p90": 0.0, "p99": 0.0}
    xs = [float(v) for v in values]
    return {"count": len(xs), "min": min(xs), "max": max(xs), "mean": sum(xs) / len(xs),
            "p50": percentile(xs, 0.5), "p90": percentile(xs, 0.9), "p99": percentile(xs, 0.99)}


def recomputed_prompt_tokens(records: Sequence[Mapping[str, object]]) -> int:
    return sum(max(0, int(r.get("prompt_tokens", 0)) - int(r.get("cached_tokens", 0))) for r in records)


def summarize_online_run(run: Mapping[str, object]) -> dict[str, object]:
    """``run``: ``{"duration_s", "requests": [...per-request records...], "scheduler_metrics"?}``."""
    duration = float(run.get("duration_s", 0.0))
    if not isfinite(duration) or duration <= 0:
        raise ValueError("online run duration_s must be positive and finite")
    records = run.get("requests")
    if not isinstance(records, list) or not records:
        raise ValueError("requests must be a non-empty list")
    completed = [r for r in records if r.get("finish_reason") in ("length", "eos", "finished")]
    rejected = [r for r in records if r.get("finish_reason") == "rejected"]
    cancelled = [r for r in records if r.get("finish_reason") == "cancelled"]
    if len(completed) + len(rejected) + len(cancelled) != len(records):
        raise ValueError("every online request must have a terminal finish_reason")

    def metric(name: str, *, optional: bool = False) -> list[float]:
        values = []
        for r in completed:
            v = r.get(name)
            if v is None:
                if optional or name not in r:  # a one-token request has no inter-token time; older records lack the field
                    continue
                raise ValueError(f"a completed request has no {name}")
            x = float(v)
            if not isfinite(x) or x < 0:
                raise ValueError(f"invalid request metric {name}={v!r}")
            values.append(x)
        return values

    out_tokens = sum(len(r.get("token_ids", ())) if "token_ids" in r else int(r.get("output_tokens", 0)) for r in completed)
    return {
        "schema_version": ONLINE_SUMMARY_SCHEMA_VERSION,
        "requests": {"total": len(records), "completed": len(completed), "rejected": len(rejected), "cancelled": len(cancelled)},
        "duration_s": duration,
        "output_tokens": out_tokens,
        "output_tokens_per_s": out_tokens / duration,
        "requests_per_s": len(completed) / duration,
        "queue_ms": summarize_distribution(metric("queue_ms", optional=True)),
        "ttft_ms": summarize_distribution(metric("ttft_ms", optional=True)),
        "tpot_ms": summarize_distribution(metric("tpot_ms", optional=True)),
        "e2e_ms": summarize_distribution(metric("latency_ms", optional=True)),
        "prompt_tokens": sum(int(r.get("prompt_tokens", 0)) for r in completed),
        "cached_prompt_tokens": sum(int(r.get("cached_tokens", 0)) for r in completed),
        "recomputed_prompt_tokens": recomputed_prompt_tokens(completed),
        "scheduler_metrics": dict(run.get("scheduler_metrics", {})),
    }
