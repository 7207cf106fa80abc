"""Pure scheduling decisions (reference ``prism_infer/engine/scheduler_policy.py:18-342``).

* ``FCFSPolicy``: admission (length, queue cap, largest visual span versus the chunk size),
  chunk sizing that never splits a visual span and stops at the multimodal prefix
  boundary, LIFO preemption victim, prefill / decode alternation.
* ``VisionAwarePolicy``: a heavy prefill (many vision patches) must wait for a number of
  decode batches while requests are decoding; light prefills may overtake it a bounded
  number of times.
* ``SLOAwarePolicy``: orders the waiting queue by deadline minus a cost-tier reserve
  (tier 0 short text, 1 light vision, 2 heavy vision: 120 / 250 / 700 ms).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Sequence as Seq

from .sequence import Sequence

if TYPE_CHECKING:  # pragma: no cover
    from .scheduler import Scheduler

SLO_RESERVE_MS = (120.0, 250.0, 700.0)
SLO_TEXT_TIER_TOKENS = 256


@dataclass(frozen=True)
class Admission:
    ok: bool
    reason: str = ""


class FCFSPolicy:
    name = "fcfs"

    def __init__(self, config) -> None:
        self.max_model_len = config.max_model_len
        self.max_queue_size = config.max_queue_size
        self.chunked = config.enable_chunked_prefill
        self.max_chunk = config.max_chunk_size
        self.max_batched = config.max_num_batched_tokens
        self.max_consecutive_prefill = config.max_consecutive_prefill_batches
        self.heavy_threshold = config.heavy_prefill_vision_patch_threshold

    # -- admission ---------------------------------------------------------------
    def admit(self, seq: Sequence, waiting_len: int) -> Admission:
        if len(seq) > self.max_model_len:
            return Admission(False, f"prompt of {len(seq)} tokens exceeds max_model_len {self.max_model_len}")
        if self.max_queue_size is not None and waiting_len >= self.max_queue_size:
            return Admission(False, "waiting queue is full")
        limit = min(self.max_chunk, self.max_batched) if self.chunked else self.max_batched
        widest = max((s.count for s in seq.visual_spans), default=0)
        if widest > limit:
            return Admission(False, f"visual span of {widest} tokens exceeds the prefill chunk limit {limit}")
        if not self.chunked and len(seq) > self.max_batched:
            return Admission(False, "prompt exceeds max_num_batched_tokens and chunked prefill is off")
        return Admission(True)

    # -- chunk sizing ------------------------------------------------------------
    def prefill_token_count(self, seq: Sequence, budget: int, *, stop_at_prefix: bool) -> int:
        start = seq.num_computed_tokens
        remaining = len(seq) - start
        if remaining <= 0 or budget <= 0:
            return 0
        if not self.chunked:
            return remaining if remaining <= budget else 0
        end = start + min(remaining, budget, self.max_chunk)
        boundary = seq.multimodal_prefix_boundary
        if stop_at_prefix and start < boundary < end:
            end = boundary
        for span in seq.visual_spans:
            if span.start < end < span.end:  # would split the span
                end = span.start if span.start > start else (span.end if span.end - start <= min(budget, self.max_chunk) else start)
                break
        return max(0, end - start)

    # -- preemption / alternation ---------------------------------------------------
    def pick_victim(self, running: Seq[Sequence]) -> Sequence:
        return running[-1]

    def order_waiting(self, waiting: list[Sequence], now_ns: int) -> None:
        return None

    def allow_prefill(self, sched: "Scheduler", head: Sequence | None) -> bool:
        return sched.consecutive_prefill_batches < self.max_consecutive_prefill

    def on_decode_batch(self) -> None:
        return None

    def on_prefill_batch(self, seqs: Seq[Sequence]) -> None:
        return None

    def may_admit(self, sched: "Scheduler", seq: Sequence) -> bool:
        """Checked for every waiting sequence before it joins a prefill batch."""
        return True

    def is_heavy(self, seq: Sequence) -> bool:
        return seq.vision_patch_count(seq.num_computed_tokens) >= self.heavy_threshold


class VisionAwarePolicy(FCFSPolicy):
    name = "vision_aware"

    def __init__(self, config) -> None:
        super().__init__(config)
        self.min_decode_between_heavy = config.min_decode_batches_between_heavy_prefills
        self.max_bypasses = config.max_light_prefill_bypasses_per_heavy
        self.decode_batches_since_heavy = self.min_decode_between_heavy
        self.bypasses = 0

    def order_waiting(self, waiting: list[Sequence], now_ns: int) -> None:
        """Let a light request overtake a blocked heavy head, a bounded number of times."""
        if len(waiting) < 2 or not self.is_heavy(waiting[0]):
            return
        if self.decode_batches_since_heavy >= self.min_decode_between_heavy or self.bypasses >= self.max_bypasses:
            return
        for i in range(1, len(waiting)):
            if not self.is_heavy(waiting[i]):
                waiting.insert(0, waiting.pop(i))
                self.bypasses += 1
                return

    def allow_prefill(self, sched: "Scheduler", head: Sequence | None) -> bool:
        if not super().allow_prefill(sched, head):
            return False
        if head is not None and self.is_heavy(head) and sched.num_decoding > 0:
            return self.decode_batches_since_heavy >= self.min_decode_between_heavy
        return True

    def may_admit(self, sched: "Scheduler", seq: Sequence) -> bool:
        if self.is_heavy(seq) and sched.num_decoding > 0:
            return self.decode_batches_since_heavy >= self.min_decode_between_heavy
        return True

    def on_decode_batch(self) -> None:
        self.decode_batches_since_heavy += 1

    def on_prefill_batch(self, seqs: Seq[Sequence]) -> None:
        if any(s.vision_patch_count() >= self.heavy_threshold for s in seqs):
            self.decode_batches_since_heavy = 0
            self.bypasses = 0


class SLOAwarePolicy(VisionAwarePolicy):
    name = "slo_aware"

    def cost_tier(self, seq: Sequence) -> int:
        patches = seq.vision_patch_count()
        if patches >= self.heavy_threshold:
            return 2
        if patches > 0 or len(seq) > SLO_TEXT_TIER_TOKENS:
            return 1
        return 0

    def reserve_ns(self, seq: Sequence) -> int:
        return int(SLO_RESERVE_MS[self.cost_tier(seq)] * 1e6)

    def order_waiting(self, waiting: list[Sequence], now_ns: int) -> None:
        def key(item: tuple[int, Sequence]):
            i, s = item
            if s.deadline_ns is None:
                return (1, i, 0)
            return (0, s.deadline_ns - self.reserve_ns(s), i)

        ordered = [s for _, s in sorted(enumerate(waiting), key=key)]
        waiting[:] = ordered


def make_policy(config) -> FCFSPolicy:
    return {"fcfs": FCFSPolicy, "vision_aware": VisionAwarePolicy, "slo_aware": SLOAwarePolicy}[config.scheduler_policy](config)
