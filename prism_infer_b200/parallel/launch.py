"""Process-group helpers shared by ``bench.py`` and the engine.

Two launch modes are supported: *external* (``python -m torch.distributed.run`` starts one
process per GPU; every process constructs ``LLM`` and ranks > 0 call ``serve_forever``) and
*spawned* (a single user process constructs ``LLM(tensor_parallel_size=N)``, which starts
N-1 worker processes itself, like the reference's ``engine/llm_engine.py:176-204``).
"""

from __future__ import annotations

import os


def rank_info() -> tuple[int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def launched_externally() -> bool:
    return int(os.environ.get("WORLD_SIZE", "1")) > 1


def bench_barrier(llm) -> None:
    group = getattr(llm, "runners", None)
    if hasattr(group, "barrier"):
        group.barrier()


def max_over_ranks(llm, value: float) -> float:
    """``time_decode_graph`` already returns the maximum over ranks; kept for symmetry."""
    return float(value)


def start_tensor_parallel_group(config, *, weights=None):
    from .tp_group import TensorParallelGroup

    return TensorParallelGroup(config, weights=weights)
