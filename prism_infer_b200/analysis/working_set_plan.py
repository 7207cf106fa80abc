"""Repeated-visual-context working-set workload (reference
``prism_infer/analysis/working_set_plan.py:34-947``, definitions summarised there at
``:493-530,601-646,749-820``).

Media groups are ordered by ``group_id`` = SHA-256 over their ordered media digests.  The
*population* phase sends one closed-loop request per group (question offset 0).  The
*measured* stream draws, for each of ``n`` requests, a group by inverse-CDF over weights
``1 / rank**alpha`` with ``random.Random(seed ^ 0x47524F5550)``, takes that group's next
question from a round-robin cursor that starts at offset 1 (every measured request asks a
different question than the group's previous one), and arrives at the cumulative sum of
``expovariate(rate)`` drawn from ``random.Random(seed ^ 0x4152524956414C)``.
Prompts are media-first: ``"Image 1: <image>\\nImage 2: <image>\\n...\\n"`` + a sentence that
numbers the images + the question, so the cacheable prefix ends after the last image.
"""

from __future__ import annotations

import hashlib
import random
from bisect import bisect_left
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

DEFAULT_SEED = 20260801
GROUP_SEED_MASK = 0x47524F5550
ARRIVAL_SEED_MASK = 0x4152524956414C
IMAGE_MARKER = "<image>"


@dataclass(frozen=True)
class MediaGroup:
    group_id: str
    media_digests: tuple[str, ...]
    questions: tuple[str, ...]
    dense_prefix_pages: int = 0

    @property
    def num_images(self) -> int:
        return len(self.media_digests)


def group_id_of(media_digests: Sequence[str]) -> str:
    h = hashlib.sha256()
    for d in media_digests:
        h.update(d.encode())
        h.update(b"\n")
    return h.hexdigest()


def media_first_prompt(num_images: int, question: str) -> str:
    head = "".join(f"Image {i + 1}: {IMAGE_MARKER}\n" for i in range(num_images))
    return f"{head}The images above are numbered Image 1 through Image {num_images} in order.\n{question}"


@dataclass(frozen=True)
class PlannedRequest:
    request_key: str
    group_index: int
    question_index: int
    arrival_offset_s: float
    phase: str  # "population" | "measured"


@dataclass
class WorkingSetPlan:
    groups: list[MediaGroup]
    population: list[PlannedRequest]
    measured: list[PlannedRequest]
    seed: int
    alpha: float
    rate: float
    page_budget: int
    working_set_pages: int

    def to_record(self) -> dict[str, object]:
        return {
            "seed": self.seed, "alpha": self.alpha, "rate_per_s": self.rate, "page_budget": self.page_budget,
            "working_set_pages": self.working_set_pages, "groups": len(self.groups),
            "questions": sum(len(g.questions) for g in self.groups),
            "population": [r.__dict__ for r in self.population], "measured": [r.__dict__ for r in self.measured],
        }


def select_groups(groups: Sequence[MediaGroup], page_budget: int, regime: str) -> list[MediaGroup]:
    """``fit``: longest sorted prefix within 70% of the budget; ``knee``: first prefix above
    the budget; ``pressure``: first prefix at 150% of the budget or every group."""
    ordered = sorted((g for g in groups if len(g.questions) >= 2), key=lambda g: g.group_id)
    chosen: list[MediaGroup] = []
    pages = 0
    for g in ordered:
        nxt = pages + g.dense_prefix_pages
        if regime == "fit" and nxt > 0.7 * page_budget and chosen:
            break
        chosen.append(g)
        pages = nxt
        if regime == "knee" and pages > page_budget:
            break
        if regime == "pressure" and pages >= 1.5 * page_budget:
            break
    if regime not in ("fit", "knee", "pressure", "all"):
        raise ValueError(f"unknown regime {regime!r}")
    return chosen


def build_plan(groups: Sequence[MediaGroup], *, num_requests: int = 600, alpha: float = 1.0, rate: float = 4.0,
               seed: int = DEFAULT_SEED, page_budget: int = 220) -> WorkingSetPlan:
    ordered = sorted(groups, key=lambda g: g.group_id)
    if not ordered:
        raise ValueError("at least one media group is required")
    population = [PlannedRequest(f"pop-{i:04d}", i, 0, 0.0, "population") for i in range(len(ordered))]
    weights = [1.0 / (rank + 1) ** alpha for rank in range(len(ordered))]
    total = sum(weights)
    cdf, acc = [], 0.0
    for w in weights:
        acc += w / total
        cdf.append(acc)
    rng_g = random.Random(seed ^ GROUP_SEED_MASK)
    rng_a = random.Random(seed ^ ARRIVAL_SEED_MASK)
    cursors = [1] * len(ordered)
    t = 0.0
    measured = []
    for i in range(num_requests):
        gi = min(bisect_left(cdf, rng_g.random()), len(ordered) - 1)
        qi = cursors[gi] % len(ordered[gi].questions)
        cursors[gi] += 1
        t += rng_a.expovariate(rate)
        measured.append(PlannedRequest(f"req-{i:05d}", gi, qi, t, "measured"))
    return WorkingSetPlan(list(ordered), population, measured, seed, alpha, rate, page_budget,
                          sum(g.dense_prefix_pages for g in ordered))


def synthetic_groups(num_groups: int = 42, num_questions: int = 85, *, seed: int = DEFAULT_SEED, min_images: int = 1,
                     max_images: int = 8, tokens_per_image: int = 198, page: int = 256,
                     question_tokens: tuple[int, int] = (16, 64)) -> list[MediaGroup]:
    """Groups of 1-8 synthetic images with 2-3 random-token questions each (85 in total for
    the default sizes); a question is a string of space-separated token ids."""
    rng = random.Random(seed)
    counts = [2] * num_groups
    for i in rng.sample(range(num_groups), max(0, num_questions - 2 * num_groups)):
        counts[i] = 3
    groups = []
    for gi in range(num_groups):
        n_img = rng.randint(min_images, max_images)
        digests = tuple(hashlib.sha256(f"{seed}:{gi}:{k}".encode()).hexdigest() for k in range(n_img))
        qs = tuple(" ".join(str(rng.randrange(1000, 100000)) for _ in range(rng.randint(*question_tokens)))
                   for _ in range(counts[gi]))
        prefix_tokens = n_img * (tokens_per_image + 6)
        groups.append(MediaGroup(group_id_of(digests), digests, qs, -(-prefix_tokens // page)))
    return groups


CHOICE_HINT = "Answer with the option's letter from the given choices directly."


def question_text(record: Mapping[str, Any]) -> str:
    """The text after the media of a materialised quality record: the question (its image markers rewritten to
    ``Image k`` so the media stay in front), the lettered options of a multiple-choice record and the answer hint."""
    q = record.get("question")
    if not isinstance(q, str) or not q:
        raise ValueError(f"record {record.get('sample_id')!r} has no question")
    parts = q.split(IMAGE_MARKER)
    n = len(record["media"])
    if len(parts) - 1 not in (0, n):
        raise ValueError(f"record {record.get('sample_id')!r}: {len(parts) - 1} image markers for {n} media")
    text = parts[0] + "".join(f"Image {k}{seg}" for k, seg in enumerate(parts[1:], 1))
    options = record.get("options")
    if isinstance(options, list) and options:
        text += "\n" + "\n".join(f"({chr(65 + i)}) {o}" for i, o in enumerate(options)) + "\n" + CHOICE_HINT
    return text


def groups_from_records(records: Sequence[Mapping[str, Any]]) -> tuple[list[MediaGroup], dict[str, str]]:
    """Media groups of materialised image records (``analysis/quality_materialization.py``): records with exactly the
    same ordered media form a group, groups with fewer than two questions are left out, questions keep their source
    order.  Also returns where each media file lives (digest -> path relative to the materialisation root).
    Reference: ``prism_infer/analysis/working_set_plan.py:56-197``."""
    by_media: dict[tuple[str, ...], list[str]] = {}
    paths: dict[str, str] = {}
    seen_ids: set[str] = set()
    for r in records:
        sid = str(r.get("sample_id"))
        if sid in seen_ids:
            raise ValueError(f"duplicate sample id {sid!r}")
        seen_ids.add(sid)
        media = r.get("media")
        if not isinstance(media, list) or not media:
            raise ValueError(f"record {sid!r} has no media")
        digests = []
        for m in media:
            d, rel = m.get("sha256"), m.get("materialized_path")
            if not (isinstance(d, str) and len(d) == 64 and isinstance(rel, str) and rel):
                raise ValueError(f"record {sid!r} has a media entry without digest or path")
            if paths.setdefault(d, rel) != rel:
                raise ValueError(f"media {d[:12]} is recorded under two paths")
            digests.append(d)
        by_media.setdefault(tuple(digests), []).append(question_text(r))
    groups = [MediaGroup(group_id_of(d), d, tuple(qs)) for d, qs in by_media.items() if len(qs) >= 2]
    groups.sort(key=lambda g: g.group_id)
    used = {d for g in groups for d in g.media_digests}
    return groups, {d: p for d, p in sorted(paths.items()) if d in used}
