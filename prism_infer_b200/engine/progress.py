"""Progress display for the synchronous ``generate*`` helpers (reference
``prism_infer/engine/llm_engine.py:52-80``: a tqdm bar that counts finished requests and shows
prefill and decode throughput in its postfix).

The reporter is fed from the step loop: ``observe_step`` with the step's phase, token count and
elapsed time, ``complete_request`` for every request that finished, ``close`` at the end.
Throughput is an exponential moving average per phase, so one slow step (a vision prefill
between decodes) does not erase the other phase's figure.  Without ``tqdm`` importable the
reporter prints one plain line per finished request to ``stderr``; disabled, every method is a
no-op, so the step loop calls it unconditionally.  ``enabled=None`` (the ``generate*`` default)
shows the bar only when the stream is a terminal: the reference's default of a visible bar for
interactive use, without progress lines in benchmark and server logs.
"""

from __future__ import annotations

import sys
from typing import Any, TextIO

from .contracts import Phase


class GenerationProgress:
    SMOOTHING = 0.3  # weight of the newest step in the moving averages

    def __init__(self, total: int, *, enabled: bool | None = True, desc: str = "Generating", file: TextIO | None = None,
                 bar_factory: Any = None) -> None:
        self.total = int(total)
        self._file = file if file is not None else sys.stderr
        if enabled is None:  # unset: a bar for a terminal (the reference's default), silence for a log
            enabled = bool(getattr(self._file, "isatty", lambda: False)())
        self.enabled = bool(enabled)
        self.completed = 0
        self.prefill_tok_s = 0.0
        self.decode_tok_s = 0.0
        self.prefill_tokens = 0
        self.decode_tokens = 0
        self._bar = None
        if not self.enabled:
            return
        if bar_factory is None:
            try:
                from tqdm.auto import tqdm as bar_factory  # type: ignore[no-redef]
            except Exception:  # pragma: no cover - tqdm ships with the image
                bar_factory = None
        if bar_factory is not None:
            self._bar = bar_factory(total=self.total, desc=desc, dynamic_ncols=True, file=self._file)

    def _blend(self, old: float, new: float) -> float:
        return new if old == 0.0 else (1.0 - self.SMOOTHING) * old + self.SMOOTHING * new

    def observe_step(self, phase: Phase, num_tokens: int, elapsed_seconds: float) -> None:
        if not self.enabled or num_tokens <= 0 or elapsed_seconds <= 0.0:
            return
        rate = num_tokens / elapsed_seconds
        if phase is Phase.PREFILL:
            self.prefill_tokens += num_tokens
            self.prefill_tok_s = self._blend(self.prefill_tok_s, rate)
        elif phase is Phase.DECODE:
            self.decode_tokens += num_tokens
            self.decode_tok_s = self._blend(self.decode_tok_s, rate)
        else:
            return
        if self._bar is not None:
            self._bar.set_postfix(self.postfix(), refresh=False)

    def postfix(self) -> dict[str, str]:
        return {"Prefill": f"{int(self.prefill_tok_s)}tok/s", "Decode": f"{int(self.decode_tok_s)}tok/s"}

    def complete_request(self, n: int = 1) -> None:
        if not self.enabled or n <= 0:
            return
        self.completed += n
        if self._bar is not None:
            self._bar.update(n)
        else:
            p = self.postfix()
            print(f"[{self.completed}/{self.total}] prefill {p['Prefill']} decode {p['Decode']}", file=self._file)

    def close(self) -> None:
        if self._bar is not None:
            self._bar.close()
            self._bar = None

    def __enter__(self) -> "GenerationProgress":
        return self

    def __exit__(self, *exc: Any) -> None:
        self.close()
