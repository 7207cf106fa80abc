"""Evidence and audit for a cold request followed by a multimodal prefix hit (reference
``benchmarks/trace_working_set_prefix.py:237-312`` evidence,
``benchmarks/audit_working_set_prefix_trace.py:22-114`` audit).

Two independent witnesses that a same-media, different-question request reused the stored
prefix instead of re-encoding the media:

* **counters** - the prefix-cache counters and the two requests' metrics before / between /
  after the pair (``validate_prefix_hit_evidence``): the cold request misses and stores once and
  reports no cached tokens; the second probes successfully, hits once, never falls back from a stale
  probe, runs no vision patches and reports cached tokens;
* **trace** - the names of the profiling regions nested inside the two requests' marker ranges
  (``prism::cold_request`` / ``prism::prefix_hit_request``): the cold one contains vision ranges,
  the hit contains none (``audit_prefix_trace``).  The nested names come either from a
  ``performance_profile`` record (``nested_names_from_profile``) or from the NVTX table of an
  Nsight Systems export (``nested_names_from_nvtx``).

Both fail closed: anything unexpected raises, nothing is patched up.
"""

from __future__ import annotations

from collections import Counter
from typing import Any, Mapping, Sequence

PREFIX_COUNTERS = ("probes", "probe_hits", "stale_probes", "hits", "misses", "stores", "evictions")
COMPLETED_REASONS = frozenset({"length", "eos", "stop"})
COLD_MARKER = "cold_request"
HIT_MARKER = "prefix_hit_request"


def _count(value: object, label: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ValueError(f"{label} must be a non-negative integer, got {value!r}")
    return value


def counter_deltas(before: Mapping[str, Any], after: Mapping[str, Any], *, phase: str) -> dict[str, int]:
    out = {}
    for key in PREFIX_COUNTERS:
        b, a = _count(before.get(key), f"{phase}.before.{key}"), _count(after.get(key), f"{phase}.after.{key}")
        if a < b:
            raise ValueError(f"{phase} prefix counter decreased: {key}")
        out[key] = a - b
    return out


def validate_prefix_hit_evidence(before: Mapping[str, Any], after_cold: Mapping[str, Any], after_hit: Mapping[str, Any],
                                 cold_request: Mapping[str, Any], hit_request: Mapping[str, Any], *,
                                 cold_vision_patches: int, hit_vision_patches: int) -> dict[str, Any]:
    """``before`` / ``after_*`` are prefix-cache counter snapshots, ``*_request`` the per-request
    metric records, ``*_vision_patches`` the patches the vision tower ran for each request."""
    cold = counter_deltas(before, after_cold, phase=COLD_MARKER)
    hit = counter_deltas(after_cold, after_hit, phase=HIT_MARKER)
    if cold["probe_hits"] or cold["hits"]:
        raise ValueError("cold request unexpectedly reused a multimodal prefix")
    if cold["misses"] != 1 or cold["stores"] != 1:
        raise ValueError("cold request did not miss and store exactly one multimodal prefix")
    if cold_request.get("finish_reason") not in COMPLETED_REASONS:
        raise ValueError(f"cold request did not complete: {cold_request.get('finish_reason')!r}")
    if _count(cold_request.get("cached_tokens"), "cold-request cached_tokens"):
        raise ValueError("cold request unexpectedly reported cached tokens")
    if _count(cold_vision_patches, "cold-request vision patches") == 0:
        raise ValueError("cold request ran no vision patches")
    if hit["probe_hits"] < 1:  # probed at submission, at the admission check and at allocation
        raise ValueError("second request's pre-admission probe did not find the stored prefix")
    if hit["hits"] != 1 or hit["misses"]:
        raise ValueError("second request was not exactly one realized prefix-cache hit")
    if hit["stale_probes"]:
        raise ValueError("second request fell back after a stale prefix probe")
    if _count(hit_vision_patches, "prefix-hit vision patches"):
        raise ValueError("second request ran the vision tower although its prefix was cached")
    if hit_request.get("finish_reason") not in COMPLETED_REASONS:
        raise ValueError(f"prefix-hit request did not complete: {hit_request.get('finish_reason')!r}")
    cached = _count(hit_request.get("cached_tokens"), "prefix-hit cached_tokens")
    prompt = _count(hit_request.get("prompt_tokens"), "prefix-hit prompt_tokens")
    if cached == 0:
        raise ValueError("prefix-hit request reported no actual cached tokens")
    if cached > prompt:
        raise ValueError("prefix-hit cached tokens exceed prompt tokens")
    return {"passed": True, "cold_request_counter_deltas": cold, "prefix_hit_request_counter_deltas": hit,
            "cold_request_vision_patches": cold_vision_patches, "prefix_hit_request_vision_patches": hit_vision_patches,
            "actual_cached_tokens": cached, "prompt_tokens": prompt, "cached_fraction": cached / prompt,
            "stale_probe_fallback": False}


def is_vision_range(name: str) -> bool:
    low = name.lower()
    return "vision" in low or "deepstack" in low


def nested_names_from_profile(record: Mapping[str, Any], marker: str) -> Counter:
    """Names of all regions below the single region called ``marker`` in a profile record."""
    regions = record["regions"]
    roots = [i for i, r in enumerate(regions) if r["name"] == marker]
    if len(roots) != 1:
        raise ValueError(f"expected exactly one {marker!r} region; found {len(roots)}")
    inside = {roots[0]}
    names: Counter = Counter()
    for i, r in enumerate(regions):  # start order: a parent always precedes its children
        if r.get("parent") in inside:
            inside.add(i)
            names[r["name"]] += 1
    return names


def nested_names_from_nvtx(ranges: Sequence[tuple[str, int, int]], marker: str, prefix: str = "prism::") -> Counter:
    """Same from NVTX ``(text, start, end)`` rows: ranges lying inside the single marker range."""
    roots = [(s, e) for n, s, e in ranges if n == prefix + marker]
    if len(roots) != 1:
        raise ValueError(f"expected exactly one {prefix + marker!r} NVTX range; found {len(roots)}")
    s0, e0 = roots[0]
    return Counter(n[len(prefix):] if n.startswith(prefix) else n for n, s, e in ranges
                   if s >= s0 and e <= e0 and (s, e, n) != (s0, e0, prefix + marker))


def audit_prefix_trace(cold_names: Mapping[str, int], hit_names: Mapping[str, int], evidence: Mapping[str, Any]) -> dict[str, Any]:
    cold_vision = sorted(n for n in cold_names if is_vision_range(n))
    hit_vision = sorted(n for n in hit_names if is_vision_range(n))
    hit_deltas = evidence["prefix_hit_request_counter_deltas"]
    checks = {
        "semantic_prefix_hit_passed": evidence.get("passed") is True,
        "cold_trace_contains_vision_ranges": bool(cold_vision),
        "prefix_hit_trace_contains_no_vision_or_deepstack_ranges": not hit_vision,
        "prefix_hit_ran_no_vision_patches": evidence.get("prefix_hit_request_vision_patches") == 0,
        "prefix_hit_used_cached_prefix_tokens": evidence.get("actual_cached_tokens", 0) > 0,
        "prefix_hit_had_no_stale_fallback": hit_deltas.get("stale_probes") == 0,
    }
    return {
        "record_type": "prefix_trace_audit", "passed": all(checks.values()), "checks": checks,
        "common_prefix_reuse": {k: evidence[k] for k in ("actual_cached_tokens", "prompt_tokens", "cached_fraction")},
        "cold_vision_ranges": {n: cold_names[n] for n in cold_vision},
        "prefix_hit_vision_ranges": {n: hit_names[n] for n in hit_vision},
        "cold_nested_ranges": dict(sorted(cold_names.items())),
        "prefix_hit_nested_ranges": dict(sorted(hit_names.items())),
    }
