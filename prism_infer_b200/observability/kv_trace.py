"""KV-cache event hooks (allocate / hit / evict / compact / swap); silent without a provider."""

from __future__ import annotations

from typing import Any, Callable

_provider: Callable[[str, dict[str, Any]], None] | None = None


def install_kv_trace_provider(fn: Callable[[str, dict[str, Any]], None] | None) -> None:
    global _provider
    _provider = fn


def emit_kv_event(kind: str, **fields: Any) -> None:
    if _provider is not None:
        _provider(kind, fields)
