"""Validators for the JSON records the benchmarks emit (reference
``prism_infer/analysis/benchmark_schema.py:458-483``).  Every record names its schema
version, the engine and model, the hardware, whether the data was synthetic, and carries
finite, non-negative measurements; scripts validate before writing and refuse to overwrite."""

from __future__ import annotations

import os
from math import isfinite
from typing import Any, Mapping

BENCHMARK_SCHEMA_VERSION = 1
REQUIRED_TOP_LEVEL = ("schema_version", "benchmark", "engine", "model", "hardware", "data", "config", "results")


class SchemaError(ValueError):
    pass


def _finite_numbers(value: Any, path: str) -> None:
    if isinstance(value, bool) or value is None or isinstance(value, str):
        return
    if isinstance(value, (int, float)):
        if not isfinite(float(value)):
            raise SchemaError(f"{path} is not finite")
        return
    if isinstance(value, Mapping):
        for k, v in value.items():
            if not isinstance(k, str):
                raise SchemaError(f"{path} has a non-string key {k!r}")
            _finite_numbers(v, f"{path}.{k}")
        return
    if isinstance(value, (list, tuple)):
        for i, v in enumerate(value):
            _finite_numbers(v, f"{path}[{i}]")
        return
    raise SchemaError(f"{path} has unsupported type {type(value).__name__}")


def validate_benchmark_record(record: Mapping[str, Any]) -> Mapping[str, Any]:
    if not isinstance(record, Mapping):
        raise SchemaError("benchmark record must be an object")
    missing = [k for k in REQUIRED_TOP_LEVEL if k not in record]
    if missing:
        raise SchemaError(f"benchmark record is missing {missing}")
    if record["schema_version"] != BENCHMARK_SCHEMA_VERSION:
        raise SchemaError(f"unsupported schema_version {record['schema_version']!r}")
    for key in ("benchmark", "engine", "model", "data"):
        if not isinstance(record[key], str) or not record[key]:
            raise SchemaError(f"{key} must be a non-empty string")
    for key in ("hardware", "config", "results"):
        if not isinstance(record[key], Mapping):
            raise SchemaError(f"{key} must be an object")
    _finite_numbers(record, "record")
    for name, value in record["results"].items():
        if isinstance(value, (int, float)) and not isinstance(value, bool) and name.endswith(("_ms", "_s", "_per_s", "_bytes")):
            if value < 0:
                raise SchemaError(f"results.{name} must be non-negative")
    return record


def write_record(path: str, record: Mapping[str, Any], *, overwrite: bool = False) -> None:
    import json

    validate_benchmark_record(record)
    if os.path.exists(path) and not overwrite:
        raise FileExistsError(f"refusing to overwrite {path}")
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(record, fh, indent=1, sort_keys=True)
    os.replace(tmp, path)
