"""Reader for Nsight Systems SQLite exports (``nsys export --type sqlite``): per engine step
and per named NVTX range, what the GPU did (reference ``benchmarks/analyze_nsys.py:95-727``).

The engine pushes NVTX ranges ``prism::<region>`` inside a ``performance_profile`` session.  A
range is a span of CPU time; the GPU work it caused is found by correlation id: every runtime
API call that starts inside the range (``CUPTI_ACTIVITY_KIND_RUNTIME``) is joined with the kernel,
copy or memset activity record of the same correlation id, which may execute after the CPU
range has ended.  Graph launches are joined with ``CUPTI_ACTIVITY_KIND_GRAPH_TRACE`` rows (a
graph replay is one activity record; its kernels are listed individually only when the capture
ran with ``--cuda-graph-trace=node``).

Nothing here needs Nsight Systems itself - only the exported file - so the summary can be made
on a machine without a GPU.  Times in the export are nanoseconds.
"""

from __future__ import annotations

import sqlite3
from bisect import bisect_left, bisect_right
from pathlib import Path
from typing import Any, Iterable, Sequence

NSYS_SUMMARY_SCHEMA_VERSION = 1
REQUIRED_TABLES = ("StringIds", "NVTX_EVENTS", "CUPTI_ACTIVITY_KIND_RUNTIME", "CUPTI_ACTIVITY_KIND_KERNEL")

# first match wins; fragments are matched against the lower-cased kernel name
KERNEL_CATEGORIES: tuple[tuple[str, tuple[str, ...]], ...] = (
    ("gemm_tcgen05", ("gemm_wx",)),
    ("attention_prefill", ("flash_tc", "flash_fwd")),
    ("attention_decode", ("paged_decode", "decode_merge", "decode_attn")),
    ("norm_rope_kv", ("rmsnorm", "layernorm", "qk_norm", "vit_rope", "reduce_norm_allgather")),
    ("kv_cache", ("kv_store", "kv_gather", "kv_scatter", "page_copy", "kv_compact")),
    ("activation", ("swiglu", "gelu")),
    ("embedding", ("embed", "pos_embed")),
    ("sampler", ("sample_kernel", "merge_candidates")),
    ("exchange", ("allgather", "wait_flags", "push", "nccl")),
    ("library_gemm", ("cutlass", "cublas", "sm100_", "sm90_", "ampere_", "gemm")),
    ("torch_elementwise", ("elementwise_kernel", "vectorized", "copy_kernel", "fill", "index", "cat")),
)


def kernel_category(name: str) -> str:
    low = name.lower()
    for category, fragments in KERNEL_CATEGORIES:
        if any(f in low for f in fragments):
            return category
    return "other"


def percentile(values: Sequence[float], fraction: float) -> float:
    """Linear-interpolated quantile of a non-empty sequence."""
    if not values:
        raise ValueError("percentile of an empty sequence")
    v = sorted(values)
    pos = fraction * (len(v) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (pos - lo)


def summarize(values: Sequence[float]) -> dict[str, float | int]:
    if not values:
        return {"count": 0, "total": 0.0, "mean": 0.0, "median": 0.0, "p90": 0.0, "min": 0.0, "max": 0.0}
    return {"count": len(values), "total": float(sum(values)), "mean": float(sum(values)) / len(values),
            "median": percentile(values, 0.5), "p90": percentile(values, 0.9), "min": float(min(values)),
            "max": float(max(values))}


def union_ns(intervals: Iterable[tuple[int, int]]) -> int:
    """Length of the union of half-open intervals: GPU busy time without double counting
    kernels that overlap on different streams."""
    total, cur_s, cur_e = 0, None, None
    for s, e in sorted(intervals):
        if e <= s:
            continue
        if cur_e is None or s > cur_e:
            if cur_e is not None:
                total += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    if cur_e is not None:
        total += cur_e - cur_s
    return total


def _tables(con: sqlite3.Connection) -> set[str]:
    return {r[0] for r in con.execute("SELECT name FROM sqlite_master WHERE type = 'table'")}


def _columns(con: sqlite3.Connection, table: str) -> set[str]:
    return {r[1] for r in con.execute(f"PRAGMA table_info({table})")}


def open_export(path: str | Path) -> sqlite3.Connection:
    """Read-only connection; refuses a file that lacks the tables an analysis needs."""
    con = sqlite3.connect(Path(path).resolve().as_uri() + "?mode=ro", uri=True)
    missing = [t for t in REQUIRED_TABLES if t not in _tables(con)]
    if missing:
        con.close()
        raise ValueError(f"not a CUDA + NVTX Nsight Systems export: missing tables {missing}")
    return con


def nvtx_ranges(con: sqlite3.Connection, name: str | None = None) -> list[tuple[str, int, int]]:
    """Closed push/pop ranges ``(text, start, end)`` in start order; the text may be inline or
    a reference into ``StringIds``."""
    has_text_id = "textId" in _columns(con, "NVTX_EVENTS")
    text = "coalesce(n.text, s.value)" if has_text_id else "n.text"
    join = "LEFT JOIN StringIds AS s ON n.textId = s.id" if has_text_id else ""
    rows = con.execute(f"SELECT {text}, n.start, n.end FROM NVTX_EVENTS AS n {join} "
                       f"WHERE n.end IS NOT NULL AND {text} IS NOT NULL ORDER BY n.start").fetchall()
    out = [(str(t), int(s), int(e)) for t, s, e in rows]
    return out if name is None else [r for r in out if r[0] == name]


class ActivityIndex:
    """Runtime calls sorted by start time, device activities keyed by correlation id."""

    def __init__(self, con: sqlite3.Connection) -> None:
        tables = _tables(con)
        self.runtime = [(int(s), int(e), int(c), str(n)) for s, e, c, n in con.execute(
            "SELECT r.start, r.end, r.correlationId, s.value FROM CUPTI_ACTIVITY_KIND_RUNTIME AS r "
            "JOIN StringIds AS s ON r.nameId = s.id ORDER BY r.start")]
        self._runtime_starts = [r[0] for r in self.runtime]
        kcols = _columns(con, "CUPTI_ACTIVITY_KIND_KERNEL")
        name_col = "demangledName" if "demangledName" in kcols else "shortName"
        self.kernels: dict[int, list[tuple[int, int, str]]] = {}
        for s, e, c, n in con.execute(
                f"SELECT k.start, k.end, k.correlationId, s.value FROM CUPTI_ACTIVITY_KIND_KERNEL AS k "
                f"JOIN StringIds AS s ON k.{name_col} = s.id ORDER BY k.start"):
            self.kernels.setdefault(int(c), []).append((int(s), int(e), str(n)))
        self.copies: dict[int, list[tuple[int, int, int]]] = {}
        for table in ("CUPTI_ACTIVITY_KIND_MEMCPY", "CUPTI_ACTIVITY_KIND_MEMSET"):
            if table in tables:
                size = "bytes" if "bytes" in _columns(con, table) else "0"
                for s, e, c, b in con.execute(f"SELECT start, end, correlationId, {size} FROM {table}"):
                    self.copies.setdefault(int(c), []).append((int(s), int(e), int(b or 0)))
        self.graphs: dict[int, list[tuple[int, int]]] = {}
        if "CUPTI_ACTIVITY_KIND_GRAPH_TRACE" in tables and "correlationId" in _columns(con, "CUPTI_ACTIVITY_KIND_GRAPH_TRACE"):
            for s, e, c in con.execute("SELECT start, end, correlationId FROM CUPTI_ACTIVITY_KIND_GRAPH_TRACE"):
                self.graphs.setdefault(int(c), []).append((int(s), int(e)))

    def runtime_within(self, start: int, end: int) -> list[tuple[int, int, int, str]]:
        """Runtime calls that start inside ``[start, end]``."""
        return self.runtime[bisect_left(self._runtime_starts, start):bisect_right(self._runtime_starts, end)]


def range_metrics(idx: ActivityIndex, start: int, end: int) -> dict[str, Any]:
    """GPU work caused by the CPU span ``[start, end]``."""
    calls = idx.runtime_within(start, end)
    api: dict[str, int] = {}
    kernels: list[tuple[int, int, str]] = []
    copies: list[tuple[int, int, int]] = []
    graphs: list[tuple[int, int]] = []
    launch_gap_us: list[float] = []
    for _, call_end, corr, name in calls:
        api[name] = api.get(name, 0) + 1
        ks = idx.kernels.get(corr, ())
        kernels.extend(ks)
        copies.extend(idx.copies.get(corr, ()))
        graphs.extend(idx.graphs.get(corr, ()))
        if ks and "LaunchKernel" in name and ks[0][0] >= call_end:
            launch_gap_us.append((ks[0][0] - call_end) / 1e3)

    def count(fragment: str) -> int:
        return sum(n for name, n in api.items() if fragment in name)

    busy = [(s, e) for s, e, _ in kernels] + [(s, e) for s, e, _ in copies] + graphs
    by_cat: dict[str, dict[str, float]] = {}
    for s, e, name in kernels:
        c = by_cat.setdefault(kernel_category(name), {"count": 0, "time_ms": 0.0})
        c["count"] += 1
        c["time_ms"] += (e - s) / 1e6
    first = min((s for s, _ in busy), default=None)
    last = max((e for _, e in busy), default=None)
    return {
        "cpu_range_ms": (end - start) / 1e6,
        "runtime_api_count": len(calls),
        "kernel_launch_api_count": count("LaunchKernel"),
        "graph_launch_api_count": count("GraphLaunch"),
        "memcpy_async_count": count("MemcpyAsync"),
        "stream_synchronize_count": count("StreamSynchronize"),
        "kernel_count": len(kernels),
        "kernel_time_ms": sum(e - s for s, e, _ in kernels) / 1e6,
        "graph_execution_ms": sum(e - s for s, e in graphs) / 1e6,
        "memcpy_time_ms": sum(e - s for s, e, _ in copies) / 1e6,
        "memcpy_bytes": sum(b for _, _, b in copies),
        "gpu_busy_ms": union_ns(busy) / 1e6,
        "gpu_span_ms": 0.0 if first is None else (last - first) / 1e6,
        "gpu_start_offset_us": 0.0 if first is None else (first - start) / 1e3,
        "gpu_tail_after_cpu_ms": 0.0 if last is None else max(0, last - end) / 1e6,
        "launch_to_kernel_median_us": percentile(launch_gap_us, 0.5) if launch_gap_us else 0.0,
        "launch_to_kernel_p90_us": percentile(launch_gap_us, 0.9) if launch_gap_us else 0.0,
        "kernel_categories": {k: by_cat[k] for k in sorted(by_cat)},
    }


_PHASE_FIELDS = ("cpu_range_ms", "kernel_count", "kernel_time_ms", "graph_execution_ms", "gpu_busy_ms", "runtime_api_count",
                 "kernel_launch_api_count", "graph_launch_api_count", "memcpy_async_count", "stream_synchronize_count",
                 "gpu_tail_after_cpu_ms", "launch_to_kernel_median_us")


def _phase_summary(steps: Sequence[dict[str, Any]]) -> dict[str, Any]:
    return {"steps": len(steps), **{f: summarize([float(s[f]) for s in steps]) for f in _PHASE_FIELDS}}


def top_kernels(idx: ActivityIndex, start: int, end: int, limit: int = 20) -> list[dict[str, Any]]:
    """Kernels caused by the span, grouped by name, by descending total time."""
    agg: dict[str, list[float]] = {}
    for _, _, corr, _ in idx.runtime_within(start, end):
        for s, e, name in idx.kernels.get(corr, ()):
            agg.setdefault(name, []).append((e - s) / 1e3)
    rows = [{"name": n, "category": kernel_category(n), "count": len(v), "total_us": sum(v), "mean_us": sum(v) / len(v)}
            for n, v in agg.items()]
    return sorted(rows, key=lambda r: -r["total_us"])[:limit]


def analyze_nsys_sqlite(path: str | Path, *, engine_range: str = "prism::engine.step", prefill_steps: int = 1,
                        target_ranges: Sequence[str] = (), top: int = 20) -> dict[str, Any]:
    """Summary of one capture: the first ``prefill_steps`` engine ranges are the prefill phase,
    the rest decode; every name in ``target_ranges`` is summarised over all its occurrences."""
    if prefill_steps < 0:
        raise ValueError("prefill_steps must be >= 0")
    con = open_export(path)
    try:
        idx = ActivityIndex(con)
        steps_nvtx = nvtx_ranges(con, engine_range)
        if len(steps_nvtx) <= prefill_steps:
            raise ValueError(f"capture holds {len(steps_nvtx)} {engine_range!r} ranges: not enough for "
                             f"{prefill_steps} prefill step(s) plus decode")
        raw = [range_metrics(idx, s, e) for _, s, e in steps_nvtx]
        targets = {}
        for name in target_ranges:
            found = nvtx_ranges(con, name)
            obs = [range_metrics(idx, s, e) for _, s, e in found]
            targets[name] = {"occurrences": len(obs), **({} if not obs else {f: summarize([float(o[f]) for o in obs]) for f in _PHASE_FIELDS})}
        span = (steps_nvtx[0][1], steps_nvtx[-1][2])
        return {
            "schema_version": NSYS_SUMMARY_SCHEMA_VERSION, "record_type": "nsys_profile_summary",
            "source": str(Path(path).resolve()), "engine_range": engine_range, "prefill_steps": prefill_steps,
            "raw_steps": raw,
            "phase_summary": {"prefill": _phase_summary(raw[:prefill_steps]), "decode": _phase_summary(raw[prefill_steps:])},
            "target_ranges": targets,
            "top_kernels": top_kernels(idx, span[0], span[1], top),
        }
    finally:
        con.close()
