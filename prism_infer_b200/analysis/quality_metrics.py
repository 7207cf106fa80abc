"""Answer-quality metrics used by the working-set quality study (reference
``prism_infer/analysis/quality_metrics.py``): ANLS for DocVQA-style answers and
multiple-choice letter extraction for MuirBench / MVBench-style prompts."""

from __future__ import annotations

import re
from typing import Sequence


def levenshtein(a: str, b: str) -> int:
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


def anls(prediction: str, answers: Sequence[str], threshold: float = 0.5) -> float:
    """Average normalised Levenshtein similarity against the best-matching reference."""
    p = " ".join(prediction.strip().lower().split())
    best = 0.0
    for ans in answers:
        a = " ".join(ans.strip().lower().split())
        if not a and not p:
            return 1.0
        nl = levenshtein(p, a) / max(len(p), len(a), 1)
        best = max(best, 1.0 - nl if nl < threshold else 0.0)
    return best


_CHOICE = re.compile(r"(?:^|[^A-Za-z])\(?([A-H])\)?(?:[^A-Za-z]|$)")


def parse_choice(text: str, num_options: int = 4) -> str | None:
    """First standalone option letter in the model output, e.g. ``(B)`` / ``B.`` / ``Answer: B``."""
    allowed = "ABCDEFGH"[:num_options]
    for m in _CHOICE.finditer(text.strip()):
        if m.group(1) in allowed:
            return m.group(1)
    return None


def choice_accuracy(predictions: Sequence[str], gold: Sequence[str], num_options: int = 4) -> float:
    if len(predictions) != len(gold) or not gold:
        raise ValueError("predictions and gold must be non-empty and aligned")
    return sum(parse_choice(p, num_options) == g for p, g in zip(predictions, gold)) / len(gold)
