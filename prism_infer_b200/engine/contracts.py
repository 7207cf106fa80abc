"""Immutable hand-off objects between scheduler, executor and runner (reference
``prism_infer/engine/contracts.py:48-522``)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Protocol, Sequence as Seq

from .sequence import Sequence


class Phase(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    IDLE = "idle"


@dataclass(frozen=True)
class PrefillSlice:
    """Logical token range of one sequence computed in this step."""

    start: int
    length: int

    @property
    def end(self) -> int:
        return self.start + self.length


@dataclass(frozen=True)
class KVTransferPlan:
    """Page traffic to apply before the model runs, in this order."""

    copy_prefix: tuple[tuple[int, int, int], ...] = ()   # (src page, dst page, rows)
    copy_on_write: tuple[tuple[int, int], ...] = ()       # (src page, dst page)
    swap_out: tuple[tuple[int, int], ...] = ()            # (gpu page, cpu page)
    swap_in: tuple[tuple[int, int], ...] = ()             # (cpu page, gpu page)

    @property
    def empty(self) -> bool:
        return not (self.copy_prefix or self.copy_on_write or self.swap_out or self.swap_in)


@dataclass(frozen=True)
class BatchPlan:
    phase: Phase
    seqs: tuple[Sequence, ...] = ()
    slices: tuple[PrefillSlice, ...] = ()
    kv_transfers: KVTransferPlan = field(default_factory=KVTransferPlan)
    num_tokens: int = 0
    num_vision_patches: int = 0

    def __post_init__(self) -> None:
        if self.phase is Phase.PREFILL and len(self.slices) != len(self.seqs):
            raise ValueError("a prefill plan needs one slice per sequence")

    @property
    def batch_size(self) -> int:
        return len(self.seqs)

    @property
    def is_idle(self) -> bool:
        return self.phase is Phase.IDLE or not self.seqs


@dataclass(frozen=True)
class ExecutionResult:
    """Sampled token per sequence; ``None`` for a prefill chunk that did not finish the prompt."""

    tokens: tuple[int | None, ...]
    duration_ms: float = 0.0
    compactions: int = 0


@dataclass(frozen=True)
class RequestOutput:
    request_id: int
    new_token: int | None
    finished: bool
    finish_reason: str | None = None
    token_ids: tuple[int, ...] = ()


@dataclass(frozen=True)
class StepResult:
    phase: Phase
    outputs: tuple[RequestOutput, ...] = ()
    num_tokens: int = 0

    @property
    def finished(self) -> tuple[RequestOutput, ...]:
        return tuple(o for o in self.outputs if o.finished)


class ModelRunnerLike(Protocol):
    def run_plan(self, plan: BatchPlan) -> ExecutionResult: ...
    def apply_kv_transfers(self, transfers: KVTransferPlan) -> None: ...
    def compact_kv(self, plans: Seq[Any]) -> None: ...


class MetricsSink(Protocol):
    def on_request_submitted(self, seq: Sequence) -> None: ...
    def on_request_scheduled(self, seq: Sequence) -> None: ...
    def on_tokens(self, seq: Sequence, n: int) -> None: ...
    def on_request_finished(self, seq: Sequence) -> None: ...
    def on_batch_completed(self, plan: BatchPlan, duration_ms: float, compactions: int) -> None: ...
