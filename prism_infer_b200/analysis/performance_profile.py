"""``performance_profile()``: the provider behind ``observability.profile_region``
(reference ``prism_infer/analysis/performance_profile.py:171-437``).

Inside a session every region records CPU wall time, a CUDA event pair (when CUDA is
available and ``cuda_timing`` is on), and pushes an NVTX range ``prism::<name>``; engine
steps attach phase / batch / token / patch metadata.  The session yields a validated JSON
record.  Outside a session ``profile_region`` stays a no-op.

Every ``engine.step`` region opens a step with the next id; regions inside it carry that id and, once the record is
taken, the step's phase (``prefill`` / ``decode`` / ...; regions outside any step are ``preprocess``).  The record
holds per-name statistics of the CPU and CUDA time (count / median / p90 / p99 / min / max), the same split by
phase, and the plain totals; ``validate_profile_record`` recomputes all of them from the raw regions.
"""

from __future__ import annotations

import time
from collections.abc import Mapping
from contextlib import contextmanager
from math import isfinite
from typing import Any, Iterator

import torch

from ..observability import install_profile_provider

PROFILE_SCHEMA_VERSION = 2  # 2: step ids, phases, statistical summaries
STEP_REGION = "engine.step"
STAT_KEYS = ("count", "median", "p90", "p99", "min", "max")


def _quantile(ordered: list[float], q: float) -> float:
    pos = q * (len(ordered) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(ordered) - 1)
    return ordered[lo] + (ordered[hi] - ordered[lo]) * (pos - lo)


def summarize_values(values: list[float]) -> dict[str, float | int]:
    v = sorted(float(x) for x in values)
    if not v:
        raise ValueError("no values to summarise")
    return {"count": len(v), "median": _quantile(v, 0.5), "p90": _quantile(v, 0.9), "p99": _quantile(v, 0.99), "min": v[0], "max": v[-1]}


def summarize_regions(regions: list[Mapping[str, Any]]) -> dict[str, dict[str, Any]]:
    """Per region name: calls, statistics of the CPU time and (where measured) of the CUDA time; inclusive times."""
    out: dict[str, dict[str, Any]] = {}
    for name in sorted({str(r["name"]) for r in regions}):
        rows = [r for r in regions if r["name"] == name]
        cuda = [float(r["cuda_ms"]) for r in rows if r.get("cuda_ms") is not None]
        out[name] = {"calls": len(rows), "cpu_ms": summarize_values([float(r["cpu_ms"]) for r in rows]),
                     "cuda_ms": summarize_values(cuda) if cuda else None}
    return out


def _totals(regions: list[Mapping[str, Any]]) -> dict[str, dict[str, float]]:
    totals: dict[str, dict[str, float]] = {}
    for r in regions:
        t = totals.setdefault(r["name"], {"count": 0, "cpu_ms": 0.0, "cuda_ms": 0.0})
        t["count"] += 1
        t["cpu_ms"] += r["cpu_ms"]
        t["cuda_ms"] += r.get("cuda_ms") or 0.0
    return totals


class ProfileSession:
    def __init__(self, metadata: dict[str, Any] | None, cuda_timing: bool, nvtx: bool) -> None:
        self.metadata = dict(metadata or {})
        self.cuda_timing = cuda_timing and torch.cuda.is_available()
        self.nvtx = nvtx and torch.cuda.is_available()
        self.regions: list[dict[str, Any]] = []
        self.steps: list[dict[str, Any]] = []
        self._pending: list[tuple[dict[str, Any], Any, Any]] = []
        self._open: list[int] = []  # indices (in start order) of the regions currently open
        self._t0 = time.perf_counter_ns()
        self._active_step: dict[str, Any] | None = None

    @contextmanager
    def region(self, name: str, *, cuda: bool = True, metadata: dict[str, Any] | None = None) -> Iterator[None]:
        # regions are listed in start order; "parent" is the index of the enclosing region
        rec: dict[str, Any] = {"name": name, "metadata": dict(metadata or {}), "parent": self._open[-1] if self._open else None}
        opened_step = None
        if name == STEP_REGION and self._active_step is None:
            opened_step = self._active_step = {"step_id": len(self.steps), "status": "ok"}
            self.steps.append(opened_step)
        rec["step_id"] = self._active_step["step_id"] if self._active_step is not None else None
        self.regions.append(rec)
        self._open.append(len(self.regions) - 1)
        start_ev = end_ev = None
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"prism::{name}")
        if cuda and self.cuda_timing:
            start_ev, end_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start_ev.record()
        t0 = time.perf_counter_ns()
        rec["start_ns"] = t0 - self._t0
        try:
            yield
        except BaseException:
            if opened_step is not None:
                opened_step["status"] = "error"
            raise
        finally:
            rec["cpu_ms"] = (time.perf_counter_ns() - t0) / 1e6
            if opened_step is not None:
                self._active_step = None
            self._open.pop()
            if end_ev is not None:
                end_ev.record()
                self._pending.append((rec, start_ev, end_ev))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def step(self, meta: dict[str, Any]) -> None:
        """Scheduling metadata of the step under way (phase, batch size, tokens, patches); a caller outside any
        ``engine.step`` region gets a step of its own."""
        if self._active_step is not None:
            self._active_step.update({k: v for k, v in meta.items() if k not in ("step_id", "status")})
        else:
            self.steps.append({"step_id": len(self.steps), "status": "ok", **{k: v for k, v in meta.items() if k not in ("step_id", "status")}})

    def finalize(self) -> dict[str, Any]:
        if self._pending:
            torch.cuda.synchronize()
            for rec, s, e in self._pending:
                rec["cuda_ms"] = s.elapsed_time(e)
            self._pending.clear()
        phase_of = {st["step_id"]: str(st.get("phase", "unknown")) for st in self.steps}
        for r in self.regions:
            r.setdefault("cpu_ms", 0.0)  # a region still open when the record is taken
            r.setdefault("cuda_ms", None)
            r["phase"] = "preprocess" if r["step_id"] is None else phase_of[r["step_id"]]
        phases = sorted({r["phase"] for r in self.regions})
        return {"schema_version": PROFILE_SCHEMA_VERSION, "record_type": "performance_profile", "metadata": self.metadata,
                "cuda_timing": self.cuda_timing, "regions": self.regions, "steps": self.steps, "totals": _totals(self.regions),
                "summary": summarize_regions(self.regions),
                "summary_by_phase": {p: summarize_regions([r for r in self.regions if r["phase"] == p]) for p in phases}}


@contextmanager
def performance_profile(metadata: dict[str, Any] | None = None, *, cuda_timing: bool = True,
                        nvtx: bool = True) -> Iterator[ProfileSession]:
    session = ProfileSession(metadata, cuda_timing, nvtx)
    install_profile_provider(session.region, session.step)
    try:
        yield session
    finally:
        install_profile_provider(None, None)


def _duration(value: Any, what: str, *, optional: bool) -> None:
    if value is None and optional:
        return
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not isfinite(float(value)) or value < 0:
        raise ValueError(f"profile region {what} must be a finite, non-negative number")


def validate_profile_record(record: dict[str, Any]) -> dict[str, Any]:
    """Structure of the record and every aggregate recomputed from the raw regions."""
    if record.get("schema_version") != PROFILE_SCHEMA_VERSION or record.get("record_type") != "performance_profile":
        raise ValueError("unsupported profile schema_version or record_type")
    if not isinstance(record.get("metadata"), Mapping) or not isinstance(record.get("cuda_timing"), bool):
        raise ValueError("profile record needs a metadata object and a cuda_timing flag")
    steps, regions = record.get("steps"), record.get("regions")
    if not isinstance(steps, list) or not isinstance(regions, list):
        raise ValueError("profile record needs lists of steps and regions")
    ids = set()
    for st in steps:
        sid = st.get("step_id") if isinstance(st, Mapping) else None
        if isinstance(sid, bool) or not isinstance(sid, int) or sid < 0 or sid in ids:
            raise ValueError(f"profile step ids are distinct non-negative integers, got {sid!r}")
        ids.add(sid)
        if st.get("status") not in ("ok", "error"):
            raise ValueError("profile step status is 'ok' or 'error'")
    phase_of = {st["step_id"]: str(st.get("phase", "unknown")) for st in steps}
    for i, r in enumerate(regions):
        if not isinstance(r, Mapping) or not isinstance(r.get("name"), str) or not r["name"]:
            raise ValueError("malformed region entry: no name")
        _duration(r.get("cpu_ms"), "cpu_ms", optional=False)
        _duration(r.get("cuda_ms"), "cuda_ms", optional=True)
        if not isinstance(r.get("metadata"), Mapping):
            raise ValueError("profile region metadata must be an object")
        if r.get("step_id") is not None and r["step_id"] not in ids:
            raise ValueError(f"region {r['name']!r} belongs to the unknown step {r['step_id']!r}")
        want = "preprocess" if r.get("step_id") is None else phase_of[r["step_id"]]
        if r.get("phase") != want:
            raise ValueError(f"region {r['name']!r} has phase {r.get('phase')!r}, its step says {want!r}")
        parent = r.get("parent")
        if parent is not None and not (isinstance(parent, int) and 0 <= parent < i):
            raise ValueError("a region's parent precedes it in the list")
    if record.get("summary") != summarize_regions(regions):
        raise ValueError("profile summary does not follow from the regions")
    phases = sorted({r["phase"] for r in regions})
    if record.get("summary_by_phase") != {p: summarize_regions([r for r in regions if r["phase"] == p]) for p in phases}:
        raise ValueError("profile summary by phase does not follow from the regions")
    if record.get("totals") != _totals(regions):
        raise ValueError("profile totals do not follow from the regions")
    return record
