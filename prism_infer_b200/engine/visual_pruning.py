"""Which visual tokens of a prompt keep their KV rows.

Span finding, the keep count ``max(min_keep, ceil(n * ratio))`` capped at ``n``, uniform
index selection (first and last always kept, evenly spaced ordinals between) and
score-based top-k, with the same defaults as the reference
(``prism_infer/engine/visual_pruning.py:23-30,395-519``).  A prompt whose visual tokens
are all video frames keeps everything unless a video floor is configured.
"""

from __future__ import annotations

from dataclasses import dataclass
from math import ceil, isfinite
from typing import Mapping, Sequence

DEFAULT_KEEP_RATIO = 0.6
DEFAULT_MIN_KEEP = 32


@dataclass(frozen=True)
class VisualSpan:
    start: int
    end: int  # exclusive
    modality: str  # "image" | "video"

    @property
    def count(self) -> int:
        return self.end - self.start


@dataclass(frozen=True)
class PruningConfig:
    keep_ratio: float = DEFAULT_KEEP_RATIO
    min_keep_tokens: int = DEFAULT_MIN_KEEP
    video_min_keep_tokens: int | None = None
    strategy: str = "uniform"


@dataclass(frozen=True)
class PruningDecision:
    total_visual_tokens: int
    kept: tuple[int, ...]
    dropped: tuple[int, ...]
    spans: tuple[VisualSpan, ...]
    strategy: str

    @property
    def keep_ratio_actual(self) -> float:
        return len(self.kept) / self.total_visual_tokens if self.total_visual_tokens else 1.0


def find_visual_spans(token_ids: Sequence[int], image_token_id: int, video_token_id: int) -> tuple[VisualSpan, ...]:
    spans: list[VisualSpan] = []
    i, n = 0, len(token_ids)
    while i < n:
        t = token_ids[i]
        if t == image_token_id or t == video_token_id:
            j = i
            while j < n and token_ids[j] == t:
                j += 1
            spans.append(VisualSpan(i, j, "image" if t == image_token_id else "video"))
            i = j
        else:
            i += 1
    return tuple(spans)


def target_keep_count(total: int, min_keep: int, ratio: float) -> int:
    if total <= 0:
        return 0
    if total <= min_keep:
        return total
    return min(total, max(min_keep, ceil(total * ratio)))


def uniform_keep(indices: Sequence[int], keep: int) -> tuple[int, ...]:
    n = len(indices)
    if keep >= n:
        return tuple(indices)
    if keep == 1:
        return (indices[n // 2],)
    chosen: list[int] = []
    seen: set[int] = set()
    for k in range(keep):
        o = round(k * (n - 1) / (keep - 1))
        if o not in seen:
            seen.add(o)
            chosen.append(o)
    o = 0
    while len(chosen) < keep:
        if o not in seen:
            seen.add(o)
            chosen.append(o)
        o += 1
    return tuple(indices[o] for o in sorted(chosen))


def score_keep(indices: Sequence[int], keep: int, scores: Mapping[int, float]) -> tuple[int, ...]:
    ranked = []
    for i in indices:
        if i not in scores:
            raise ValueError(f"missing score for visual token index {i}")
        s = float(scores[i])
        if not isfinite(s):
            raise ValueError(f"non-finite score for visual token index {i}")
        ranked.append((-s, i))
    ranked.sort()
    return tuple(sorted(i for _, i in ranked[:keep]))


def compute_pruning_decision(
    token_ids: Sequence[int],
    image_token_id: int,
    video_token_id: int,
    config: PruningConfig,
    *,
    end: int | None = None,
    scores: Mapping[int, float] | None = None,
) -> PruningDecision | None:
    """Decision over the visual tokens in ``token_ids[:end]``; ``None`` when there are none."""
    spans = find_visual_spans(token_ids[: end if end is not None else len(token_ids)], image_token_id, video_token_id)
    indices = [i for s in spans for i in range(s.start, s.end)]
    if not indices:
        return None
    if all(s.modality == "video" for s in spans):
        floor = len(indices) if config.video_min_keep_tokens is None else config.video_min_keep_tokens
    else:
        floor = config.min_keep_tokens
    keep = target_keep_count(len(indices), floor, config.keep_ratio)
    if config.strategy == "uniform":
        kept = uniform_keep(indices, keep)
    elif config.strategy in ("score", "attention"):
        if scores is None:
            raise ValueError("score-based pruning requires token scores keyed by token index")
        kept = score_keep(indices, keep, scores)
    else:
        raise ValueError(f"unsupported strategy {config.strategy!r}")
    kept_set = set(kept)
    return PruningDecision(len(indices), kept, tuple(i for i in indices if i not in kept_set), spans, config.strategy)


def retained_positions(prefix_len: int, decision: PruningDecision | None) -> tuple[int, ...]:
    """Every non-visual position below ``prefix_len`` plus the kept visual positions."""
    if decision is None:
        return tuple(range(prefix_len))
    dropped = set(decision.dropped)
    return tuple(p for p in range(prefix_len) if p not in dropped)


class RuntimeVisualTokenScorer:
    """Query-aware scores for the ``attention`` strategy (reference
    ``prism_infer/engine/visual_pruning.py:73-195``): in each chosen decoder layer, the attention
    that the LAST query of every sequence pays to each of its visual tokens - softmax over all of
    the sequence's keys, mean over query heads - summed over the layers and averaged at the end.

    ``observe`` takes the step's flattened ``q [T, Hq_local, D]`` and ``k [T, Hkv_local, D]`` (after
    QK-norm and rotary) and keeps device tensors only; ``finalize`` averages over layers, sums the
    ranks' head means through ``reduce_sum`` (every rank holds ``Hq / world`` heads) and moves the
    result to the host once.  ``rows`` gives each sequence's ``(seq_id, first row, row count,
    visual token indices relative to the sequence)``; a sequence must be present with its whole
    prompt, because the last query has to see every key."""

    def __init__(self, rows: Sequence[tuple[int, int, int, Sequence[int]]], layer_ids: Sequence[int]) -> None:
        self.layer_ids = tuple(sorted({int(i) for i in layer_ids}))
        if not self.layer_ids or self.layer_ids[0] < 0:
            raise ValueError(f"layer_ids must be non-empty and non-negative: {list(layer_ids)}")
        self.rows = tuple((int(s), int(lo), int(n), tuple(int(v) for v in vis)) for s, lo, n, vis in rows)
        self.total_tokens = max((lo + n for _, lo, n, _ in self.rows), default=0)
        self._sums: dict[int, object] = {}
        self._seen: set[int] = set()

    def observe(self, layer_id: int, q, k, scale: float) -> None:
        import torch

        if layer_id not in self.layer_ids:
            return
        if layer_id in self._seen:
            raise RuntimeError(f"layer {layer_id} observed twice")
        if q.dim() != 3 or k.dim() != 3 or q.shape[2] != k.shape[2] or q.shape[1] % k.shape[1]:
            raise ValueError(f"expected q [T, Hq, D] and k [T, Hkv, D] with Hq a multiple of Hkv, got {list(q.shape)} and {list(k.shape)}")
        if q.shape[0] < self.total_tokens or k.shape[0] < self.total_tokens:
            raise ValueError(f"scorer covers {self.total_tokens} rows, got q {q.shape[0]} and k {k.shape[0]}")
        groups = q.shape[1] // k.shape[1]
        for seq_id, lo, n, vis in self.rows:
            if not vis:
                continue
            q_last = q[lo + n - 1].float()                                   # [Hq, D]
            keys = k[lo:lo + n].float()                                      # [n, Hkv, D]
            logits = torch.einsum("hgd,thd->hgt", q_last.view(k.shape[1], groups, -1), keys) * float(scale)
            probs = torch.softmax(logits, dim=-1).mean(dim=(0, 1))           # [n]
            picked = probs.index_select(0, torch.tensor(vis, dtype=torch.long, device=probs.device))
            self._sums[seq_id] = picked if seq_id not in self._sums else self._sums[seq_id] + picked
        self._seen.add(layer_id)

    def finalize(self, *, world_size: int = 1, reduce_sum=None) -> dict[int, dict[int, float]]:
        missing = sorted(set(self.layer_ids) - self._seen)
        if missing:
            raise RuntimeError(f"scorer did not observe layers {missing}")
        out: dict[int, dict[int, float]] = {}
        for seq_id, _, _, vis in self.rows:
            if not vis:
                out[seq_id] = {}
                continue
            scores = self._sums[seq_id] / len(self._seen)
            if world_size > 1:
                if reduce_sum is None:
                    raise ValueError("a tensor-parallel scorer needs reduce_sum")
                scores = reduce_sum(scores.contiguous()) / world_size
            out[seq_id] = dict(zip(vis, (float(v) for v in scores.cpu().tolist())))
        return out
