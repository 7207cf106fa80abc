"""Request lifecycle: an audited finite-state machine.

WAITING -> PREFILLING -> DECODING <-> SWAPPED -> FINISHED, with CANCELLED reachable from
every live state and REJECTED only from WAITING (reference
``prism_infer/engine/request.py:50-176``).  Preemption by recompute sends a PREFILLING or
DECODING request back to WAITING.
"""

from __future__ import annotations

import enum
import itertools
import threading
from dataclasses import dataclass, field


class RequestState(enum.Enum):
    WAITING = "waiting"
    PREFILLING = "prefilling"
    DECODING = "decoding"
    SWAPPED = "swapped"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    REJECTED = "rejected"

    @property
    def terminal(self) -> bool:
        return self in (RequestState.FINISHED, RequestState.CANCELLED, RequestState.REJECTED)


_S = RequestState
ALLOWED_TRANSITIONS: dict[RequestState, frozenset[RequestState]] = {
    _S.WAITING: frozenset({_S.PREFILLING, _S.CANCELLED, _S.REJECTED}),
    _S.PREFILLING: frozenset({_S.PREFILLING, _S.DECODING, _S.FINISHED, _S.WAITING, _S.SWAPPED, _S.CANCELLED}),
    _S.DECODING: frozenset({_S.DECODING, _S.SWAPPED, _S.WAITING, _S.FINISHED, _S.CANCELLED}),
    _S.SWAPPED: frozenset({_S.DECODING, _S.PREFILLING, _S.WAITING, _S.CANCELLED}),
    _S.FINISHED: frozenset(),
    _S.CANCELLED: frozenset(),
    _S.REJECTED: frozenset(),
}


class InvalidTransition(RuntimeError):
    pass


@dataclass
class RequestLifecycle:
    request_id: int
    state: RequestState = RequestState.WAITING
    finish_reason: str | None = None
    history: list[tuple[RequestState, RequestState, str]] = field(default_factory=list)

    def transition(self, new: RequestState, reason: str = "") -> None:
        if new not in ALLOWED_TRANSITIONS[self.state]:
            raise InvalidTransition(f"request {self.request_id}: {self.state.value} -> {new.value} ({reason})")
        self.history.append((self.state, new, reason))
        self.state = new
        if new.terminal:
            self.finish_reason = reason or new.value


class RequestIdAllocator:
    """Monotonic, thread-safe request ids."""

    def __init__(self, start: int = 0) -> None:
        self._it = itertools.count(start)
        self._lock = threading.Lock()

    def __call__(self) -> int:
        with self._lock:
            return next(self._it)
