"""Grouping of quality samples by identical ordered visual context, media-first prompts and
the paired dense / compact comparison of the working-set quality study (behaviour of the
reference's ``prism_infer/analysis/working_set_quality.py:157-345``).
"""

from __future__ import annotations

from collections import defaultdict
from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from typing import Any

from .identity import canonical_json_sha256
from .schema_constants import SHA256_HEX_LENGTH, is_lower_hex


@dataclass(frozen=True)
class GroupedQualitySample:
    record: Mapping[str, Any]
    media_group_id: str
    question_index: int
    group_size: int


def ordered_media_sha256(record: Mapping[str, Any]) -> tuple[str, ...]:
    media = record.get("media")
    if not isinstance(media, list) or not media:
        raise ValueError("quality record must contain a non-empty media list")
    digests = tuple(m.get("sha256") if isinstance(m, Mapping) else None for m in media)
    if not all(is_lower_hex(d, SHA256_HEX_LENGTH) for d in digests):
        raise ValueError("quality record media SHA-256 identities are invalid")
    return digests  # type: ignore[return-value]


def media_group_id(record: Mapping[str, Any], *, sampling_identity: Mapping[str, Any] | None = None) -> str:
    bound = record.get("temporal_bound")
    if bound is not None and not isinstance(bound, Mapping):
        raise ValueError("temporal_bound must be a mapping or None")
    return canonical_json_sha256({"ordered_media_sha256": list(ordered_media_sha256(record)),
                                  "temporal_bound": None if bound is None else {str(k): bound[k] for k in sorted(bound)},
                                  "sampling_identity": None if sampling_identity is None else dict(sampling_identity)})


def select_multi_question_groups(records: Sequence[Mapping[str, Any]], *, max_groups: int | None = None,
                                 sampling_identity: Mapping[str, Any] | None = None) -> list[GroupedQualitySample]:
    """Groups of at least two questions over exactly the same ordered media, ordered by group
    digest; inside a group the source order is kept (so "first question" is well defined)."""
    if max_groups is not None and max_groups <= 0:
        raise ValueError("max_groups must be positive or None")
    groups: dict[str, list[Mapping[str, Any]]] = defaultdict(list)
    for r in records:
        groups[media_group_id(r, sampling_identity=sampling_identity)].append(r)
    chosen = sorted(g for g, rs in groups.items() if len(rs) >= 2)
    if max_groups is not None:
        chosen = chosen[:max_groups]
    return [GroupedQualitySample(r, g, i, len(groups[g])) for g in chosen for i, r in enumerate(groups[g])]


def build_media_first_prompt(question: str, n_images: int, *, marker: str = "<image>", options: Sequence[str] = (),
                             hint: str = "") -> str:
    """``Image 1: <image>\\n ... Image N: <image>\\n`` + a sentence naming the numbering + the
    question with its markers rewritten to ``Image k``; the visual prefix is then identical for
    every question of a group."""
    if n_images <= 0:
        raise ValueError("n_images must be positive")
    parts = question.split(marker)
    if len(parts) - 1 not in (0, n_images):
        raise ValueError(f"question has {len(parts) - 1} image markers, expected 0 or {n_images}")
    rewritten = parts[0] + "".join(f"Image {k}{seg}" for k, seg in enumerate(parts[1:], 1))
    head = "".join(f"Image {k}: {marker}\n" for k in range(1, n_images + 1))
    body = f"The images above are numbered Image 1 through Image {n_images} in order.\n{rewritten}"
    if options:
        body += "\n" + "\n".join(options)
    if hint:
        body += "\n" + hint
    return head + body


def summarize_stage_samples(samples: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
    n = len(samples)
    correct = sum(1 for s in samples if s.get("correct"))
    deleted = [int(s.get("deleted_visual_tokens", 0)) for s in samples]
    return {"samples": n, "correct": correct, "accuracy": correct / n if n else 0.0,
            "samples_with_deletions": sum(1 for d in deleted if d > 0), "deleted_visual_tokens": sum(deleted)}


def paired_deleted_subset(dense: Sequence[Mapping[str, Any]], compact: Sequence[Mapping[str, Any]]) -> dict[str, Any]:
    """Accuracy of both arms on the samples whose visual tokens the compact arm actually deleted
    (the cohort the reference reports, e.g. 27/49 -> 20/49)."""
    by_id = {s["sample_id"]: s for s in dense}
    if set(by_id) != {s["sample_id"] for s in compact}:
        raise ValueError("dense and compact arms cover different samples")
    cohort = [s for s in compact if int(s.get("deleted_visual_tokens", 0)) > 0]
    return {"cohort": len(cohort), "dense_correct": sum(1 for s in cohort if by_id[s["sample_id"]].get("correct")),
            "compact_correct": sum(1 for s in cohort if s.get("correct"))}
