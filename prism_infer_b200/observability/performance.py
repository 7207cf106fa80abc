"""``profile_region``: dependency-inverted hook for CPU / CUDA-event / NVTX timing."""

from __future__ import annotations

from contextlib import nullcontext
from typing import Any, Callable, ContextManager

_provider: Callable[..., ContextManager] | None = None
_step_provider: Callable[[dict[str, Any]], None] | None = None
_NULL = nullcontext()


def install_profile_provider(region: Callable[..., ContextManager] | None,
                             step: Callable[[dict[str, Any]], None] | None = None) -> None:
    global _provider, _step_provider
    _provider, _step_provider = region, step


def profile_region(name: str, *, cuda: bool = True, metadata: dict[str, Any] | None = None) -> ContextManager:
    if _provider is None:
        return _NULL
    return _provider(name, cuda=cuda, metadata=metadata)


def profile_step_metadata(meta: dict[str, Any]) -> None:
    if _step_provider is not None:
        _step_provider(meta)
