"""Validators for the JSON records the benchmarks emit (reference
``prism_infer/analysis/benchmark_schema.py:458-483`` and the per-part validators before it).
Every record names its schema version, the engine and model, the hardware, whether the data was
synthetic, and carries finite, non-negative measurements.  On top of that each benchmark has a
contract: the fields its ``config`` and ``results`` (or every row of a results list) must carry,
with their kinds, and the relations between them that a well-formed run satisfies (a p99 is not
below its p50, a cache cannot hit more often than it was asked, tokens per second follow from
the step time).  Scripts validate before writing and refuse to overwrite."""

from __future__ import annotations

import os
from math import isfinite
from typing import Any, Mapping

BENCHMARK_SCHEMA_VERSION = 2  # 2: per-benchmark contracts
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
    if record["schema_version"] not in (1, BENCHMARK_SCHEMA_VERSION):
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
    contract = CONTRACTS.get(record["benchmark"])
    if contract is not None:
        contract(record)
    return record


# ---- per-benchmark contracts ---------------------------------------------------------------------------
# kind of a field: "pos" (> 0), "nonneg" (>= 0), "posint", "count" (integer >= 0), "frac" (0..1), "str", "bool",
# "obj" (mapping), "list"; a trailing "?" makes the field optional.
def _check_kind(value: Any, kind: str, path: str) -> None:
    number = isinstance(value, (int, float)) and not isinstance(value, bool)
    ok = {
        "pos": number and value > 0, "nonneg": number and value >= 0,
        "posint": isinstance(value, int) and not isinstance(value, bool) and value > 0,
        "count": isinstance(value, int) and not isinstance(value, bool) and value >= 0,
        "frac": number and 0 <= value <= 1, "str": isinstance(value, str) and bool(value), "bool": isinstance(value, bool),
        "obj": isinstance(value, Mapping), "list": isinstance(value, (list, tuple)),
    }[kind]
    if not ok:
        raise SchemaError(f"{path} = {value!r} is not a valid {kind}")


def _check_fields(obj: Any, fields: Mapping[str, str], path: str) -> None:
    if not isinstance(obj, Mapping):
        raise SchemaError(f"{path} must be an object")
    for name, kind in fields.items():
        optional = kind.endswith("?")
        if name not in obj:
            if optional:
                continue
            raise SchemaError(f"{path}.{name} is missing")
        _check_kind(obj[name], kind.rstrip("?"), f"{path}.{name}")


def _close(a: float, b: float, rel: float = 0.02) -> bool:
    return abs(a - b) <= rel * max(abs(a), abs(b), 1e-12)


def _decode_matrix(record: Mapping[str, Any]) -> None:
    _check_fields(record["config"], {"workload": "str", "output_tokens": "posint", "tp": "posint", "kv": "str"}, "config")
    rows = record["results"].get("rows")
    _check_kind(rows, "list", "results.rows")
    seen = set()
    for i, row in enumerate(rows):
        path = f"results.rows[{i}]"
        _check_fields(row, {"batch": "posint", "ttft_ms_mean": "pos", "ttft_ms_max": "pos", "tpot_ms_mean": "pos", "output_tok_per_s": "pos",
                            "preprocess_ms": "nonneg", "steady_step_ms_median": "pos?", "steady_tok_per_s": "pos?"}, path)
        if row["batch"] in seen:
            raise SchemaError(f"{path}.batch {row['batch']} appears twice")
        seen.add(row["batch"])
        if row["ttft_ms_max"] < row["ttft_ms_mean"] * (1 - 1e-9):
            raise SchemaError(f"{path}: the largest TTFT is below the mean")
        if ("steady_step_ms_median" in row) != ("steady_tok_per_s" in row):
            raise SchemaError(f"{path}: steady step time and steady throughput come together")
        if "steady_step_ms_median" in row and not _close(row["steady_tok_per_s"], row["batch"] * 1e3 / row["steady_step_ms_median"]):
            raise SchemaError(f"{path}: steady_tok_per_s does not follow from batch and steady_step_ms_median")
    if record["hardware"].get("gpus") != record["config"]["tp"]:
        raise SchemaError("hardware.gpus and config.tp disagree")


def _media_cache_reuse(record: Mapping[str, Any]) -> None:
    _check_fields(record["config"], {"case": "str", "batch": "posint", "mode": "str", "max_tokens": "posint"}, "config")
    cells = record["results"].get("cells")
    _check_kind(cells, "list", "results.cells")
    for i, cell in enumerate(cells):
        path = f"results.cells[{i}]"
        _check_fields(cell, {"repeat_rate": "frac", "requests": "posint", "wall_s": "pos", "requests_per_s": "pos", "output_tokens": "count",
                             "visual_embedding_cache": "obj", "prefix_cache": "obj"}, path)
        _check_fields(cell["visual_embedding_cache"], {"hits": "count", "misses": "count"}, f"{path}.visual_embedding_cache")
        _check_fields(cell["prefix_cache"], {"hits": "count", "misses": "count", "stores": "count", "evictions": "count"}, f"{path}.prefix_cache")
        if not _close(cell["requests_per_s"], cell["requests"] / cell["wall_s"]):
            raise SchemaError(f"{path}: requests_per_s does not follow from requests and wall_s")
        if cell["output_tokens"] > cell["requests"] * record["config"]["max_tokens"]:
            raise SchemaError(f"{path}: more output tokens than the requests may produce")


def _online_working_set(record: Mapping[str, Any]) -> None:
    cfg, res = record["config"], record["results"]
    _check_fields(cfg, {"variant": "str", "groups": "posint", "questions": "posint", "requests": "posint", "rate_per_s": "pos", "pages": "posint",
                        "page_tokens": "posint", "kv_budget_bytes": "posint", "working_set_pages": "count", "max_tokens": "posint", "tp": "posint"},
                  "config")
    _check_fields(res, {"ttft_p50_ms": "pos", "ttft_p99_ms": "pos", "e2e_p50_ms": "pos", "e2e_p99_ms": "pos", "recomputed_prompt_tokens": "count",
                        "prompt_tokens": "posint", "output_tokens_per_s": "pos", "completed": "count", "duration_s": "pos", "resident_media": "count",
                        "prefix_evictions": "count", "prefix_hits": "count", "resident_pages": "count"}, "results")
    for lo, hi in (("ttft_p50_ms", "ttft_p99_ms"), ("e2e_p50_ms", "e2e_p99_ms"), ("ttft_p50_ms", "e2e_p50_ms"), ("ttft_p99_ms", "e2e_p99_ms")):
        if res[hi] < res[lo] * (1 - 1e-9):
            raise SchemaError(f"results.{hi} is below results.{lo}")
    if res["recomputed_prompt_tokens"] > res["prompt_tokens"]:
        raise SchemaError("more prompt tokens recomputed than submitted")
    if res["completed"] > cfg["requests"]:
        raise SchemaError("more requests completed than were sent")
    if res["resident_pages"] > cfg["pages"]:
        raise SchemaError("the prefix cache holds more pages than the KV budget has")
    if res["resident_media"] > cfg["groups"]:
        raise SchemaError("more media resident than the workload has groups")


def _system_mode_matrix(record: Mapping[str, Any]) -> None:
    _check_fields(record["config"], {"mode": "str", "workload": "str", "tp": "posint"}, "config")
    res = record["results"]
    _check_fields(res, {"ttft_ms": "pos", "tpot_ms": "nonneg", "e2e_ms": "pos", "output_tokens_per_s": "pos", "batch": "posint"}, "results")
    if res["e2e_ms"] < res["ttft_ms"] * (1 - 1e-9):
        raise SchemaError("results.e2e_ms is below results.ttft_ms")


CONTRACTS = {
    "decode_matrix": _decode_matrix,
    "media_cache_reuse": _media_cache_reuse,
    "online_working_set": _online_working_set,
    "system_mode_matrix": _system_mode_matrix,
}


def write_record(path: str, record: Mapping[str, Any], *, overwrite: bool = False) -> None:
    import json

    validate_benchmark_record(record)
    if os.path.exists(path) and not overwrite:
        raise FileExistsError(f"refusing to overwrite {path}")
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as fh:
        json.dump(record, fh, indent=1, sort_keys=True)
    os.replace(tmp, path)
