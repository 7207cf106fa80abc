"""Sampler module (reference ``prism_infer/layers/sampler.py:10-55``).

One token per row of the logits: arg-max where the row's temperature is zero (lowest id wins a
tie), otherwise a draw from ``softmax(logits / temperature)`` by the exponential race
(``argmax(p / e)`` with ``e ~ Exp(1)``).  On CUDA the whole batch - greedy, random or mixed -
is one launch of the fused sampling kernel, whose noise is a counter-based hash of
``(seed, step, row, column)``; there is no split into a greedy and a random sub-batch and no
host synchronisation to find out which rows are which.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops

SAMPLING_NUMERICAL_EPSILON = 1.0e-10
SAMPLING_MODES = frozenset({"greedy", "random", "mixed"})


class Sampler(nn.Module):
    def __init__(self, seed: int = 0) -> None:
        super().__init__()
        self.seed = int(seed)
        self._calls = 0  # advances the noise stream from call to call

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor | None, *, sampling_mode: str | None = None,
                step: torch.Tensor | None = None) -> torch.Tensor:
        if sampling_mode is not None and sampling_mode not in SAMPLING_MODES:
            raise ValueError(f"unsupported sampling mode: {sampling_mode!r}")
        logits = logits.float().contiguous()
        if sampling_mode == "greedy":
            return ops.sample(logits, None)
        if temperatures is None:
            raise ValueError("temperatures are required for non-greedy sampling")
        temperatures = temperatures.to(device=logits.device, dtype=torch.float32)
        if sampling_mode == "random":
            # every row is drawn: a zero temperature is lifted to the smallest positive one
            temperatures = temperatures.clamp_min(SAMPLING_NUMERICAL_EPSILON)
        else:
            temperatures = torch.where(temperatures <= SAMPLING_NUMERICAL_EPSILON, torch.zeros_like(temperatures), temperatures)
        if step is None:
            step = torch.full((1,), self._calls, dtype=torch.int64, device=logits.device)
            self._calls += 1
        return ops.sample(logits, temperatures, seed=self.seed, step=step)
