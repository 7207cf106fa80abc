"""``model_type`` -> model family (reference ``prism_infer/models/model_registry.py:10-35``).
Only the Qwen3-VL family is implemented; an unknown type fails at start-up with the list of
known ones rather than somewhere inside weight loading."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


@dataclass(frozen=True)
class ModelFamily:
    name: str
    multimodal: bool
    architecture_from_config: Callable[[Any], Any]
    model_class_path: str  # "module:Class", imported on demand


def _qwen3_vl_arch(cfg: Any):
    from .architecture import Qwen3VLArch

    return Qwen3VLArch.from_hf_config(cfg)


_FAMILIES = {
    "qwen3_vl": ModelFamily("qwen3_vl", True, _qwen3_vl_arch, "prism_infer_b200.models.qwen3_vl:Qwen3VLModel"),
}


def known_model_types() -> list[str]:
    return sorted(_FAMILIES)


def resolve_model_family(model_type: str) -> ModelFamily:
    try:
        return _FAMILIES[model_type]
    except KeyError:
        raise ValueError(f"unsupported model_type {model_type!r}; supported: {known_model_types()}") from None


def load_model_class(family: ModelFamily):
    import importlib

    module, _, cls = family.model_class_path.partition(":")
    return getattr(importlib.import_module(module), cls)
