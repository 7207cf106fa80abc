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


# ---- MVBench (multiple-choice video questions) -------------------------------------------------------
# Prompt layout and answer extraction follow the public lmms-eval task (``tasks/mvbench/utils.py``, the
# ``mcq_acc`` metric), which the reference reproduces in ``prism_infer/analysis/quality_metrics.py:205-246``:
# the prompt spells "Option" in the singular and ends with the instruction below; the extractor accepts a
# leading "B. text" answer, else strips VQA-style punctuation and takes the first standalone letter A-E.
MVBENCH_INSTRUCTION = "Only give the best option.\n"
MVBENCH_LABELS = "ABCDE"
_VQA_PUNCTUATION = (";", "/", "[", "]", '"', "{", "}", "(", ")", "=", "+", "\\", "_", "-", ">", "<", "@", "`", ",", "?", "!")
_LEADING_ANSWER = re.compile(r"^([A-E])\.\s*(.+)$", re.IGNORECASE)
_DIGIT_COMMA_DIGIT = re.compile(r"(\d)(,)(\d)")
_PERIOD_NOT_IN_NUMBER = re.compile(r"(?!<=\d)(\.)(?!\d)")   # the upstream pattern, kept as published (its look-behind is a literal)
_STANDALONE_LABEL = re.compile(r"\b([A-E])\b", re.IGNORECASE)


def mvbench_prompt(question: str, candidates: Sequence[str]) -> str:
    """``Question:...`` / ``Option:`` / one ``(A) candidate`` line per candidate / the instruction."""
    if not isinstance(question, str) or not question:
        raise ValueError("an MVBench question is a non-empty string")
    if not 2 <= len(candidates) <= len(MVBENCH_LABELS) or not all(isinstance(c, str) for c in candidates):
        raise ValueError("MVBench takes two to five string candidates")
    lines = "".join(f"({label}) {cand}\n" for label, cand in zip(MVBENCH_LABELS, candidates))
    return f"Question:{question}\nOption:\n{lines}{MVBENCH_INSTRUCTION}"


def mvbench_choice(response: str) -> tuple[str | None, str]:
    """``(label or None, how it was found)`` for a model answer to an MVBench prompt."""
    if not isinstance(response, str):
        raise TypeError("an MVBench response is a string")
    lead = _LEADING_ANSWER.match(response.strip())
    if lead:
        return lead.group(1).upper(), "leading_label_period"
    flat = response.replace("\n", " ").replace("\t", " ").strip()
    text = flat
    for mark in _VQA_PUNCTUATION:
        glued = f"{mark} " in flat or f" {mark}" in flat or _DIGIT_COMMA_DIGIT.search(flat) is not None
        text = text.replace(mark, "" if glued else " ")
    text = _PERIOD_NOT_IN_NUMBER.sub("", text).strip().strip("'").strip('"').strip(")").strip("(").lower()
    found = _STANDALONE_LABEL.search(text)
    return (found.group(1).upper(), "embedded_label") if found else (None, "unparseable")


def mvbench_score(record: dict, prediction: str) -> dict:
    """Per-sample trace: target label, parsed label, how it was parsed, 0 / 1 score, whether anything was answered.
    ``record`` carries ``candidates`` and ``answer_index``."""
    label, how = mvbench_choice(prediction)
    target = MVBENCH_LABELS[int(record["answer_index"])]
    if not 0 <= int(record["answer_index"]) < len(record["candidates"]):
        raise ValueError("answer_index is outside the candidates")
    return {"target": target, "prediction": label, "parse_method": how, "score": int(label == target), "answered": bool(prediction.strip())}


def mvbench_accuracy(samples: Sequence[dict]) -> dict:
    """Aggregate recomputed from per-sample traces only: accuracy over all samples and the answered fraction."""
    if not samples:
        return {"samples": 0}
    n = len(samples)
    return {"samples": n, "accuracy": sum(int(s["score"]) for s in samples) / n, "answered": sum(bool(s["answered"]) for s in samples) / n,
            "unparseable": sum(s["prediction"] is None for s in samples)}
