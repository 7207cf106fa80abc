"""Validator for the quality-data protocol file: which model revision, which dataset
revisions and which deterministic sample selection a quality run used (reference:
``prism_infer/analysis/quality_protocol.py:15-117``).  It checks identities only; it holds no
pass thresholds.
"""

from __future__ import annotations

import json
from collections.abc import Mapping
from pathlib import Path
from typing import Any

from .schema_constants import GIT_REVISION_HEX_LENGTH, is_lower_hex

QUALITY_PROTOCOL_SCHEMA_VERSION = 2
QUALITY_MATERIALIZATION_STATUSES = frozenset({"pending", "materialized", "conditional_manual_media", "excluded"})
_DATASET_STRINGS = ("category", "source", "repository", "split", "sample_id_field", "metric")


class _Path:
    """Typed accessors that name the JSON path in their error messages."""

    def __init__(self, obj: Mapping[str, Any], where: str) -> None:
        if not isinstance(obj, Mapping):
            raise ValueError(f"{where} must be an object")
        self.obj, self.where = obj, where

    def get(self, key: str, kind: type | tuple[type, ...], what: str) -> Any:
        v = self.obj.get(key)
        if isinstance(v, bool) and kind is not bool or not isinstance(v, kind):
            raise ValueError(f"{self.where}.{key} must be {what}")
        return v

    def string(self, key: str) -> str:
        v = self.get(key, str, "a non-empty string")
        if not v:
            raise ValueError(f"{self.where}.{key} must be a non-empty string")
        return v

    def positive(self, key: str) -> int:
        v = self.get(key, int, "a positive integer")
        if v <= 0:
            raise ValueError(f"{self.where}.{key} must be a positive integer")
        return v

    def revision(self, key: str) -> str:
        v = self.string(key)
        if not is_lower_hex(v, GIT_REVISION_HEX_LENGTH):
            raise ValueError(f"{self.where}.{key} must be a 40-digit lowercase hexadecimal revision")
        return v

    def child(self, key: str) -> "_Path":
        return _Path(self.get(key, Mapping, "an object"), f"{self.where}.{key}")


def validate_quality_protocol(protocol: Mapping[str, Any]) -> None:
    root = _Path(protocol, "protocol")
    if protocol.get("schema_version") != QUALITY_PROTOCOL_SCHEMA_VERSION:
        raise ValueError("unsupported quality protocol schema_version")
    root.string("name")
    model = root.child("model")
    model.revision("revision")
    model.revision("processor_revision")
    sel = root.child("selection")
    sel.string("algorithm")
    sel.positive("seed")
    sel.get("materialization_requires_media_sha256", bool, "a boolean")
    datasets = root.get("datasets", list, "a non-empty list")
    if not datasets:
        raise ValueError("protocol.datasets must be a non-empty list")
    seen: set[str] = set()
    for i, entry in enumerate(datasets):
        d = _Path(entry, f"protocol.datasets[{i}]")
        ident = d.string("id")
        if ident in seen:
            raise ValueError(f"duplicate quality dataset id {ident!r}")
        seen.add(ident)
        for key in _DATASET_STRINGS:
            d.string(key)
        d.revision("revision")
        if d.positive("development_samples") > d.positive("final_samples"):
            raise ValueError(f"{d.where}.development_samples exceeds final_samples")
        status = d.string("materialization_status")
        if status not in QUALITY_MATERIALIZATION_STATUSES:
            raise ValueError(f"{d.where}.materialization_status is unsupported: {status!r}")


def load_quality_protocol(path: str | Path) -> dict[str, Any]:
    with Path(path).open("r", encoding="utf-8") as fh:
        protocol = json.load(fh)
    validate_quality_protocol(protocol)
    return protocol
