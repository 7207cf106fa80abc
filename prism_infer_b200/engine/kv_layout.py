"""Logical versus physical KV length of a sequence, and the validated compaction plan.

After visual-token compaction the first ``logical_prefix_len`` prompt tokens are
represented by fewer physical KV rows: ``retained_positions`` lists, in order, the original
token positions whose rows were kept.  RoPE was applied with logical positions when the
rows were written, so attention only needs physical lengths; the scheduler and the input
preparer translate between the two with this descriptor (reference
``prism_infer/engine/kv_layout.py:18-285``).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class KVLayout:
    logical_prefix_len: int
    retained_positions: tuple[int, ...]

    def __post_init__(self) -> None:
        if self.logical_prefix_len < 0:
            raise ValueError("logical_prefix_len must be non-negative")
        prev = -1
        for p in self.retained_positions:
            if not prev < p < self.logical_prefix_len:
                raise ValueError("retained_positions must be strictly increasing and inside the prefix")
            prev = p

    @property
    def physical_prefix_len(self) -> int:
        return len(self.retained_positions)

    @property
    def dropped(self) -> int:
        return self.logical_prefix_len - len(self.retained_positions)

    def physical_len(self, logical_len: int) -> int:
        if logical_len < self.logical_prefix_len:
            raise ValueError("logical length shorter than the compacted prefix")
        return logical_len - self.dropped

    def physical_index(self, logical_index: int) -> int:
        """Physical row of a token at or beyond the compacted prefix."""
        if logical_index < self.logical_prefix_len:
            raise ValueError("token lies inside the compacted prefix")
        return logical_index - self.dropped

    def validate_block_table(self, logical_len: int, num_blocks: int, page: int) -> None:
        need = -(-self.physical_len(logical_len) // page)
        if num_blocks < need:
            raise ValueError(f"block table has {num_blocks} pages, layout needs {need}")

    def record(self) -> dict:
        return {"logical_prefix_len": self.logical_prefix_len, "retained_positions": list(self.retained_positions)}

    @classmethod
    def from_record(cls, rec: dict) -> "KVLayout":
        return cls(int(rec["logical_prefix_len"]), tuple(int(p) for p in rec["retained_positions"]))


@dataclass(frozen=True)
class CompactionPlan:
    """Move retained rows to the dense front of the sequence's own page table.

    ``src_slots[i] -> dst_slots[i]`` are flat slots (``block * page + offset``);
    ``released_blocks`` become free once the device copy has finished.
    """

    seq_id: int
    layout: KVLayout
    src_slots: tuple[int, ...]
    dst_slots: tuple[int, ...]
    kept_blocks: tuple[int, ...]
    released_blocks: tuple[int, ...]
    block_table_version: int

    def __post_init__(self) -> None:
        if len(self.src_slots) != len(self.dst_slots):
            raise ValueError("source and destination slot lists differ in length")
        if len(self.src_slots) < self.layout.physical_prefix_len:
            raise ValueError("plan must move every retained row (plus any rows computed behind the prefix)")
        if len(set(self.dst_slots)) != len(self.dst_slots):
            raise ValueError("destination slots must be unique")
        if set(self.kept_blocks) & set(self.released_blocks):
            raise ValueError("a page cannot be both kept and released")

    @property
    def moved_rows(self) -> int:
        return sum(1 for s, d in zip(self.src_slots, self.dst_slots) if s != d)
