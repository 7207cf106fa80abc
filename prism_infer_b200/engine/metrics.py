"""Thread-safe per-request and per-batch metrics ledger (reference
``prism_infer/engine/metrics.py:17-231``): queue time, TTFT, mean TPOT, inter-token
latencies, end-to-end latency, cached tokens, finish reason; batch phase / size / tokens /
patches / duration / compactions."""

from __future__ import annotations

import collections
import threading
import time
from dataclasses import dataclass, field
from typing import Callable

from .contracts import BatchPlan
from .sequence import Sequence


@dataclass
class RequestMetrics:
    request_id: int
    prompt_tokens: int
    submitted_ns: int
    scheduled_ns: int | None = None
    first_token_ns: int | None = None
    last_token_ns: int | None = None
    finished_ns: int | None = None
    cached_tokens: int = 0
    output_tokens: int = 0
    finish_reason: str | None = None
    dropped_prompt_tokens: int = 0   # visual tokens whose K / V rows a compacting mode removed from the cache
    inter_token_ms: list[float] = field(default_factory=list)

    def record(self) -> dict[str, object]:
        ms = lambda a, b: None if a is None or b is None else (b - a) / 1e6  # noqa: E731
        tpot = sum(self.inter_token_ms) / len(self.inter_token_ms) if self.inter_token_ms else None
        return {
            "request_id": self.request_id, "prompt_tokens": self.prompt_tokens, "cached_tokens": self.cached_tokens,
            "output_tokens": self.output_tokens, "queue_ms": ms(self.submitted_ns, self.scheduled_ns),
            "ttft_ms": ms(self.submitted_ns, self.first_token_ns), "tpot_ms": tpot,
            "inter_token_ms": list(self.inter_token_ms), "latency_ms": ms(self.submitted_ns, self.finished_ns),
            "finish_reason": self.finish_reason, "dropped_prompt_tokens": self.dropped_prompt_tokens,
        }


class EngineMetrics:
    """``max_records`` bounds the ledger of a long-running server: the oldest batch records and
    the oldest request records are dropped beyond it (a decode step adds a batch record every few
    milliseconds).  Benchmarks reset the ledger between phases and never reach the bound."""

    def __init__(self, clock_ns: Callable[[], int] = time.perf_counter_ns, max_records: int = 200_000) -> None:
        self._clock = clock_ns
        self._lock = threading.Lock()
        self.max_records = max_records
        self.requests: dict[int, RequestMetrics] = {}
        self.batches: collections.deque[dict[str, object]] = collections.deque(maxlen=max_records)

    def reset(self) -> None:
        with self._lock:
            self.requests.clear()
            self.batches.clear()

    def on_request_submitted(self, seq: Sequence) -> None:
        with self._lock:
            t = seq.arrival_ns if seq.arrival_ns is not None else self._clock()
            self.requests[seq.seq_id] = RequestMetrics(seq.seq_id, seq.num_prompt_tokens, t)
            while len(self.requests) > self.max_records:
                self.requests.pop(next(iter(self.requests)))  # insertion order: the oldest request

    def on_request_scheduled(self, seq: Sequence) -> None:
        with self._lock:
            m = self.requests.get(seq.seq_id)
            if m is not None and m.scheduled_ns is None:
                m.scheduled_ns = self._clock()
                m.cached_tokens = seq.num_cached_tokens

    def on_tokens(self, seq: Sequence, n: int = 1) -> None:
        with self._lock:
            m = self.requests.get(seq.seq_id)
            if m is None:
                return
            now = self._clock()
            if m.first_token_ns is None:
                m.first_token_ns = now
            elif m.last_token_ns is not None:
                m.inter_token_ms.append((now - m.last_token_ns) / 1e6 / max(1, n))
            m.last_token_ns = now
            m.output_tokens += n
            m.dropped_prompt_tokens = max(m.dropped_prompt_tokens, int(seq.dropped_tokens))  # the layout is gone once the request finishes

    def on_request_finished(self, seq: Sequence) -> None:
        with self._lock:
            m = self.requests.get(seq.seq_id)
            if m is not None:
                m.finished_ns = self._clock()
                m.finish_reason = seq.lifecycle.finish_reason

    def on_batch_completed(self, plan: BatchPlan, duration_ms: float, compactions: int = 0) -> None:
        with self._lock:
            self.batches.append({
                "phase": plan.phase.value, "batch_size": plan.batch_size, "tokens": plan.num_tokens,
                "vision_patches": plan.num_vision_patches, "duration_ms": duration_ms, "compactions": compactions,
            })

    def snapshot(self) -> dict[str, object]:
        with self._lock:
            return {"requests": [m.record() for m in self.requests.values()], "batches": list(self.batches)}

    def recent_finished(self, limit: int = 2048) -> list[dict[str, object]]:
        """Records of the newest ``limit`` finished requests, newest first (a cheap view for periodic summaries: the full
        snapshot of a long-running server copies every record)."""
        out: list[dict[str, object]] = []
        with self._lock:
            for m in reversed(self.requests.values()):
                if m.finished_ns is not None:
                    out.append(m.record())
                    if len(out) >= limit:
                        break
        return out


class NullMetrics:
    def on_request_submitted(self, seq): ...
    def on_request_scheduled(self, seq): ...
    def on_tokens(self, seq, n=1): ...
    def on_request_finished(self, seq): ...
    def on_batch_completed(self, plan, duration_ms, compactions=0): ...
    def reset(self): ...
    def snapshot(self): return {"requests": [], "batches": []}
    def recent_finished(self, limit=2048): return []
