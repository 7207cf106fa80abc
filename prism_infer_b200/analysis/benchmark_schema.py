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

BENCHMARK_SCHEMA_VERSION = 3  # 2: per-benchmark contracts; 3: system records carry execution, correctness and KV evidence
SUPPORTED_SCHEMA_VERSIONS = (1, 2, 3)
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
    if record["schema_version"] not in SUPPORTED_SCHEMA_VERSIONS:
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


STAT_KEYS = ("count", "median", "p90", "p99", "min", "max")


def _check_stats(stats: Any, path: str, *, count: int | None = None) -> None:
    """count / median / p90 / p99 / min / max of one measured quantity, in order."""
    _check_fields(stats, {"count": "posint", "median": "nonneg", "p90": "nonneg", "p99": "nonneg", "min": "nonneg", "max": "nonneg"}, path)
    if count is not None and stats["count"] != count:
        raise SchemaError(f"{path}.count is {stats['count']}, the run had {count} rounds")
    ladder = [stats[k] for k in ("min", "median", "p90", "p99", "max")]
    if any(hi < lo * (1 - 1e-9) for lo, hi in zip(ladder, ladder[1:])):
        raise SchemaError(f"{path}: min <= median <= p90 <= p99 <= max does not hold")


def _int_keyed_counts(obj: Any, path: str) -> dict[int, int]:
    if not isinstance(obj, Mapping):
        raise SchemaError(f"{path} must be an object")
    out = {}
    for k, v in obj.items():
        if not (isinstance(k, str) and k.isdigit() and int(k) > 0):
            raise SchemaError(f"{path} has the key {k!r}; keys are positive batch sizes")
        _check_kind(v, "count", f"{path}.{k}")
        out[int(k)] = v
    return out


def _execution_evidence(ex: Any) -> None:
    """Which path each decode step took.  Graph mode: a step of batch size n replays the smallest captured bucket
    that holds n, steps beyond the largest bucket run eagerly; eager mode: no replay at all (reference
    ``prism_infer/analysis/benchmark_schema.py:684-927``)."""
    _check_fields(ex, {"backend": "str", "graph_batch_sizes": "list", "decode_batch_sizes": "obj", "graph_replays": "obj",
                       "eager_decode_steps": "count", "decode_steps": "count"}, "execution")
    if ex["backend"] not in ("eager", "cuda_graph"):
        raise SchemaError(f"execution.backend {ex['backend']!r} is neither 'eager' nor 'cuda_graph'")
    buckets = list(ex["graph_batch_sizes"])
    if any(isinstance(b, bool) or not isinstance(b, int) or b <= 0 for b in buckets) or buckets != sorted(set(buckets)):
        raise SchemaError("execution.graph_batch_sizes must be ascending positive integers without repeats")
    sizes = _int_keyed_counts(ex["decode_batch_sizes"], "execution.decode_batch_sizes")
    replays = _int_keyed_counts(ex["graph_replays"], "execution.graph_replays")
    if sum(sizes.values()) != ex["decode_steps"]:
        raise SchemaError("execution.decode_steps is not the sum of execution.decode_batch_sizes")
    if ex["backend"] == "eager":
        if buckets or any(replays.values()):
            raise SchemaError("an eager run captured or replayed graphs")
        if ex["eager_decode_steps"] != ex["decode_steps"]:
            raise SchemaError("an eager run has decode steps that did not run eagerly")
        return
    if not buckets:
        raise SchemaError("a cuda_graph run captured no graph")
    if set(replays) - set(buckets):
        raise SchemaError("execution.graph_replays names a batch size that was not captured")
    want = {b: 0 for b in buckets}
    eager = 0
    for n, c in sizes.items():
        if n > buckets[-1]:
            eager += c
        else:
            want[next(b for b in buckets if b >= n)] += c
    if eager != ex["eager_decode_steps"] or any(replays.get(b, 0) != c for b, c in want.items()):
        raise SchemaError(f"execution: the decode batch sizes imply replays {want} and {eager} eager steps, "
                          f"the record has {dict(sorted(replays.items()))} and {ex['eager_decode_steps']}")


def _correctness_evidence(c: Any, *, batch: int) -> None:
    from .identity import canonical_json_sha256

    _check_fields(c, {"requests": "posint", "output_tokens": "posint", "output_token_ids": "list", "output_token_ids_sha256": "str",
                      "identical_across_repeats": "bool"}, "correctness")
    ids = c["output_token_ids"]
    if c["requests"] != batch or len(ids) != batch:
        raise SchemaError("correctness: one token-id list per request of the batch is required")
    for i, row in enumerate(ids):
        if not isinstance(row, (list, tuple)) or len(row) != c["output_tokens"] or \
                any(isinstance(t, bool) or not isinstance(t, int) or t < 0 for t in row):
            raise SchemaError(f"correctness.output_token_ids[{i}] must hold {c['output_tokens']} non-negative token ids")
    if canonical_json_sha256([list(r) for r in ids]) != c["output_token_ids_sha256"]:
        raise SchemaError("correctness.output_token_ids_sha256 does not match the token ids")
    if not c["identical_across_repeats"]:
        raise SchemaError("greedy decoding of the same inputs gave different tokens in different rounds")


def _kv_accounting(kv: Any, *, batch: int) -> None:
    _check_fields(kv, {"mode": "str", "page_tokens": "posint", "pages": "count", "bytes_per_page": "posint", "prompt_tokens": "list",
                       "dropped_prompt_tokens": "list", "dense_prompt_bytes": "posint", "active_prompt_bytes": "posint"}, "kv_cache")
    prompt, dropped = kv["prompt_tokens"], kv["dropped_prompt_tokens"]
    if len(prompt) != batch or len(dropped) != batch:
        raise SchemaError("kv_cache: one prompt length and one dropped-token count per request")
    for i, (n, d) in enumerate(zip(prompt, dropped)):
        _check_kind(n, "posint", f"kv_cache.prompt_tokens[{i}]")
        _check_kind(d, "count", f"kv_cache.dropped_prompt_tokens[{i}]")
        if d >= n:
            raise SchemaError(f"kv_cache: request {i} dropped {d} of {n} prompt tokens")
    page, per = kv["page_tokens"], kv["bytes_per_page"]
    if kv["dense_prompt_bytes"] != sum(-(-n // page) for n in prompt) * per:
        raise SchemaError("kv_cache.dense_prompt_bytes does not follow from the prompt lengths, the page size and the bytes per page")
    if kv["active_prompt_bytes"] != sum(-(-(n - d) // page) for n, d in zip(prompt, dropped)) * per:
        raise SchemaError("kv_cache.active_prompt_bytes does not follow from the resident prompt tokens")
    compacting = kv["mode"].startswith("visual_compact")
    if any(dropped) and not compacting:
        raise SchemaError(f"kv_cache: mode {kv['mode']!r} does not compact, yet prompt tokens were dropped")


def _system_mode_matrix(record: Mapping[str, Any]) -> None:
    _check_fields(record["config"], {"mode": "str", "workload": "str", "tp": "posint", "repeats": "posint?", "output_tokens": "posint?"}, "config")
    res = record["results"]
    _check_fields(res, {"ttft_ms": "pos", "tpot_ms": "nonneg", "e2e_ms": "pos", "output_tokens_per_s": "pos", "batch": "posint"}, "results")
    if res["e2e_ms"] < res["ttft_ms"] * (1 - 1e-9):
        raise SchemaError("results.e2e_ms is below results.ttft_ms")
    if record["schema_version"] < 3:  # earlier records carry the four headline numbers only
        return
    _check_fields(record["config"], {"repeats": "posint", "output_tokens": "posint"}, "config")
    stats = res.get("stats")
    _check_fields(stats, {k: "obj" for k in ("ttft_ms", "tpot_ms", "e2e_ms", "output_tokens_per_s")}, "results.stats")
    for name in ("ttft_ms", "tpot_ms", "e2e_ms", "output_tokens_per_s"):
        _check_stats(stats[name], f"results.stats.{name}", count=record["config"]["repeats"])
        if not _close(res[name], stats[name]["median"], rel=1e-9):
            raise SchemaError(f"results.{name} is not the median of its rounds")
    for part in ("execution", "correctness", "kv_cache"):
        if part not in record:
            raise SchemaError(f"benchmark record is missing {part!r}")
    _execution_evidence(record["execution"])
    graph_mode = record["config"].get("enforce_eager") is False
    if "enforce_eager" in record["config"] and graph_mode != (record["execution"]["backend"] == "cuda_graph"):
        raise SchemaError("execution.backend contradicts config.enforce_eager")
    _correctness_evidence(record["correctness"], batch=res["batch"])
    if record["correctness"]["output_tokens"] != record["config"]["output_tokens"]:
        raise SchemaError("correctness.output_tokens and config.output_tokens disagree")
    _kv_accounting(record["kv_cache"], batch=res["batch"])


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
