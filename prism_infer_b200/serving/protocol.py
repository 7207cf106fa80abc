"""Framework-independent wire types of the serving layer (reference
``prism_infer/serving/protocol.py:16-102``): a validated ``GenerationRequest`` and the
``ServingEvent`` stream (accepted, token, done, error)."""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any

from ..sampling_params import SamplingParams


class Modality(str, Enum):
    TEXT = "text"
    IMAGE = "image"
    VIDEO = "video"


class EventKind(str, Enum):
    ACCEPTED = "accepted"
    TOKEN = "token"
    DONE = "done"
    ERROR = "error"


@dataclass(frozen=True)
class GenerationRequest:
    request_id: str
    prompt: str
    modality: Modality
    media: Any | tuple[Any, ...] | None
    sampling_params: SamplingParams
    ttft_slo_ms: float | None = None  # time-to-first-token target from arrival; used by the SLO-aware scheduler policy

    def __post_init__(self) -> None:
        for broken, error in _REQUEST_RULES:
            if broken(self):
                raise error[0](error[1].format(modality=getattr(self.modality, "value", self.modality)))


def _blank(value: object) -> bool:
    return not isinstance(value, str) or not value.strip()


# (violation predicate, (exception type, message)) in the order the fields are checked
_REQUEST_RULES = (
    (lambda r: _blank(r.request_id), (ValueError, "request_id must be a non-empty string")),
    (lambda r: _blank(r.prompt), (ValueError, "prompt must be a non-empty string")),
    (lambda r: not isinstance(r.modality, Modality), (TypeError, "modality must be a Modality")),
    (lambda r: not isinstance(r.sampling_params, SamplingParams), (TypeError, "sampling_params must be SamplingParams")),
    (lambda r: r.modality is Modality.TEXT and r.media is not None, (ValueError, "text requests must not include media")),
    (lambda r: r.modality is not Modality.TEXT and r.media is None, (ValueError, "{modality} requests require media")),
    (lambda r: isinstance(r.media, tuple) and len(r.media) == 0, (ValueError, "media tuples must not be empty")),
    (lambda r: r.ttft_slo_ms is not None and not (0.0 < float(r.ttft_slo_ms) < float("inf")),
     (ValueError, "ttft_slo_ms must be a finite positive number")),
)


@dataclass(frozen=True)
class ServingEvent:
    request_id: str
    kind: EventKind
    engine_request_id: int | None = None
    token_id: int | None = None
    token_text: str | None = None
    token_ids: tuple[int, ...] = ()
    text: str | None = None
    finish_reason: str | None = None
    error: str | None = None
    prompt_tokens: int | None = None  # DONE only, when the engine can tell: the prompt's length after expansion of the media

    def to_dict(self) -> dict[str, object]:
        out: dict[str, object] = {"request_id": self.request_id, "event": self.kind.value}
        for name in ("engine_request_id", "token_id", "token_text", "text", "finish_reason", "error", "prompt_tokens"):
            value = getattr(self, name)
            if value is not None:
                out[name] = value
        if self.kind is EventKind.DONE:
            out["token_ids"] = list(self.token_ids)
        return out
