"""HTTP / SSE serving layer: ``prism-serve`` CLI, FastAPI app, engine-owner runtime."""

from .protocol import EventKind, GenerationRequest, Modality, ServingEvent
from .runtime import DuplicateRequest, IngressFull, RuntimeUnavailable, ServingRuntime

__all__ = ["EventKind", "GenerationRequest", "Modality", "ServingEvent", "ServingRuntime", "IngressFull",
           "DuplicateRequest", "RuntimeUnavailable"]
