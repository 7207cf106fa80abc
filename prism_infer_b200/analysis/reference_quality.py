"""Free-text answer scores against reference strings: token F1 and ROUGE-L F1.

Same definitions as the reference (``prism_infer/analysis/reference_quality.py:20-100``):
text is case-folded and split into maximal runs of Unicode letters / digits; token F1 is the
harmonic mean of multiset precision and recall; ROUGE-L uses the longest common subsequence
of the two token lists.  Two empty strings score 1, one empty string scores 0.
"""

from __future__ import annotations

import re
from collections import Counter
from collections.abc import Mapping, Sequence
from typing import Any

REFERENCE_QUALITY_SCHEMA_VERSION = 1
_WORD = re.compile(r"[^\W_]+", flags=re.UNICODE)


def normalize_reference_text(text: str) -> list[str]:
    if not isinstance(text, str):
        raise ValueError("text must be a string")
    return _WORD.findall(text.casefold())


def _f1(overlap: int, n_pred: int, n_ref: int) -> float:
    if n_pred == 0 and n_ref == 0:
        return 1.0
    if overlap == 0 or n_pred == 0 or n_ref == 0:
        return 0.0
    p, r = overlap / n_pred, overlap / n_ref
    return 2.0 * p * r / (p + r)


def token_f1(prediction: str, reference: str) -> float:
    p, r = normalize_reference_text(prediction), normalize_reference_text(reference)
    return _f1(sum((Counter(p) & Counter(r)).values()), len(p), len(r))


def lcs_length(a: Sequence[str], b: Sequence[str]) -> int:
    if len(a) < len(b):
        a, b = b, a
    row = [0] * (len(b) + 1)
    for x in a:
        diag = 0
        for j, y in enumerate(b, 1):
            diag, row[j] = row[j], (diag + 1 if x == y else max(row[j], row[j - 1]))
    return row[-1]


def rouge_l_f1(prediction: str, reference: str) -> float:
    p, r = normalize_reference_text(prediction), normalize_reference_text(reference)
    return _f1(lcs_length(p, r), len(p), len(r))


def score_reference_text(prediction: str, references: Sequence[str]) -> dict[str, float]:
    """Best score over the accepted references, each metric maximised separately."""
    if not references:
        raise ValueError("at least one reference is required")
    return {"token_f1": max(token_f1(prediction, r) for r in references),
            "rouge_l_f1": max(rouge_l_f1(prediction, r) for r in references),
            "exact_match": float(any(normalize_reference_text(prediction) == normalize_reference_text(r) for r in references))}


def score_reference_batch(predictions: Mapping[str, str], references: Mapping[str, Sequence[str]]) -> dict[str, Any]:
    """Per-sample scores and their means; the two mappings must have the same sample ids."""
    if set(predictions) != set(references):
        missing = sorted(set(references) - set(predictions))
        extra = sorted(set(predictions) - set(references))
        raise ValueError(f"sample ids differ: missing={missing[:5]} unexpected={extra[:5]}")
    samples = {k: score_reference_text(predictions[k], references[k]) for k in sorted(predictions)}
    n = max(1, len(samples))
    mean = {m: sum(s[m] for s in samples.values()) / n for m in ("token_f1", "rouge_l_f1", "exact_match")}
    return {"schema_version": REFERENCE_QUALITY_SCHEMA_VERSION, "sample_count": len(samples), "mean": mean, "samples": samples}
