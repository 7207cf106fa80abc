"""``performance_profile()``: the provider behind ``observability.profile_region``
(reference ``prism_infer/analysis/performance_profile.py:171-437``).

Inside a session every region records CPU wall time, a CUDA event pair (when CUDA is
available and ``cuda_timing`` is on), and pushes an NVTX range ``prism::<name>``; engine
steps attach phase / batch / token / patch metadata.  The session yields a validated JSON
record.  Outside a session ``profile_region`` stays a no-op.
"""

from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Any, Iterator

import torch

from ..observability import install_profile_provider

PROFILE_SCHEMA_VERSION = 1


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

    @contextmanager
    def region(self, name: str, *, cuda: bool = True, metadata: dict[str, Any] | None = None) -> Iterator[None]:
        # regions are listed in start order; "parent" is the index of the enclosing region
        rec: dict[str, Any] = {"name": name, "metadata": dict(metadata or {}), "parent": self._open[-1] if self._open else None}
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
        finally:
            rec["cpu_ms"] = (time.perf_counter_ns() - t0) / 1e6
            self._open.pop()
            if end_ev is not None:
                end_ev.record()
                self._pending.append((rec, start_ev, end_ev))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def step(self, meta: dict[str, Any]) -> None:
        self.steps.append(dict(meta))

    def finalize(self) -> dict[str, Any]:
        if self._pending:
            torch.cuda.synchronize()
            for rec, s, e in self._pending:
                rec["cuda_ms"] = s.elapsed_time(e)
            self._pending.clear()
        totals: dict[str, dict[str, float]] = {}
        for r in self.regions:
            r.setdefault("cpu_ms", 0.0)  # a region still open when the record is taken
            t = totals.setdefault(r["name"], {"count": 0, "cpu_ms": 0.0, "cuda_ms": 0.0})
            t["count"] += 1
            t["cpu_ms"] += r["cpu_ms"]
            t["cuda_ms"] += r.get("cuda_ms", 0.0)
        return {"schema_version": PROFILE_SCHEMA_VERSION, "metadata": self.metadata, "regions": self.regions,
                "steps": self.steps, "totals": totals}


@contextmanager
def performance_profile(metadata: dict[str, Any] | None = None, *, cuda_timing: bool = True,
                        nvtx: bool = True) -> Iterator[ProfileSession]:
    session = ProfileSession(metadata, cuda_timing, nvtx)
    install_profile_provider(session.region, session.step)
    try:
        yield session
    finally:
        install_profile_provider(None, None)


def validate_profile_record(record: dict[str, Any]) -> dict[str, Any]:
    if record.get("schema_version") != PROFILE_SCHEMA_VERSION:
        raise ValueError("unsupported profile schema_version")
    for key in ("metadata", "regions", "steps", "totals"):
        if key not in record:
            raise ValueError(f"profile record is missing {key}")
    for r in record["regions"]:
        if "name" not in r or "cpu_ms" not in r or r["cpu_ms"] < 0:
            raise ValueError("malformed region entry")
    return record
