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

    def __post_init__(self) -> None:
        if not isinstance(self.request_id, str) or not self.request_id.strip():
            raise ValueError("request_id must be a non-empty string")
        if not isinstance(self.prompt, str) or not self.prompt.strip():
            raise ValueError("prompt must be a non-empty string")
        if not isinstance(self.modality, Modality):
            raise TypeError("modality must be a Modality")
        if not isinstance(self.sampling_params, SamplingParams):
            raise TypeError("sampling_params must be SamplingParams")
        if self.modality is Modality.TEXT and self.media is not None:
            raise ValueError("text requests must not include media")
        if self.modality is not Modality.TEXT and self.media is None:
            raise ValueError(f"{self.modality.value} requests require media")
        if isinstance(self.media, tuple) and not self.media:
            raise ValueError("media tuples must not be empty")


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

    def to_dict(self) -> dict[str, object]:
        out: dict[str, object] = {"request_id": self.request_id, "event": self.kind.value}
        for name in ("engine_request_id", "token_id", "token_text", "text", "finish_reason", "error"):
            value = getattr(self, name)
            if value is not None:
                out[name] = value
        if self.kind is EventKind.DONE:
            out["token_ids"] = list(self.token_ids)
        return out
