"""Page allocators: a reference-counted GPU pool with a content-hash index, and a CPU
swap-page pool with all-or-nothing allocation (reference
``prism_infer/engine/block_pool.py:17-267``)."""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field


class OutOfBlocks(RuntimeError):
    pass


@dataclass
class Block:
    block_id: int
    ref_count: int = 0
    hash: int | None = None
    token_ids: tuple[int, ...] = field(default_factory=tuple)

    def reset(self) -> None:
        self.ref_count = 1
        self.hash = None
        self.token_ids = ()


class GpuBlockPool:
    """Reference-counted pages.  A page whose count drops to zero returns to the free list
    but keeps its hash until it is handed out again, so a later identical prefix can
    revive it without recomputation."""

    def __init__(self, num_blocks: int) -> None:
        self.blocks = [Block(i) for i in range(num_blocks)]
        self.free: deque[int] = deque(range(num_blocks))
        self.hash_to_block: dict[int, int] = {}

    @property
    def num_blocks(self) -> int:
        return len(self.blocks)

    @property
    def num_free(self) -> int:
        return len(self.free)

    @property
    def num_used(self) -> int:
        return len(self.blocks) - len(self.free)

    def allocate(self) -> int:
        if not self.free:
            raise OutOfBlocks("no free GPU page")
        bid = self.free.popleft()
        blk = self.blocks[bid]
        if blk.hash is not None and self.hash_to_block.get(blk.hash) == bid:
            del self.hash_to_block[blk.hash]
        blk.reset()
        return bid

    def allocate_many(self, n: int) -> list[int]:
        if n > len(self.free):
            raise OutOfBlocks(f"need {n} GPU pages, {len(self.free)} free")
        return [self.allocate() for _ in range(n)]

    def retain(self, bid: int) -> None:
        blk = self.blocks[bid]
        if blk.ref_count == 0:
            self.free.remove(bid)  # revive a cached page
        blk.ref_count += 1

    def release(self, bid: int) -> None:
        blk = self.blocks[bid]
        if blk.ref_count <= 0:
            raise RuntimeError(f"page {bid} released more often than retained")
        blk.ref_count -= 1
        if blk.ref_count == 0:
            self.free.append(bid)

    def lookup(self, h: int, token_ids: tuple[int, ...]) -> int | None:
        bid = self.hash_to_block.get(h)
        if bid is None or self.blocks[bid].token_ids != token_ids:
            return None
        return bid

    def publish(self, bid: int, h: int, token_ids: tuple[int, ...]) -> None:
        blk = self.blocks[bid]
        blk.hash, blk.token_ids = h, token_ids
        self.hash_to_block[h] = bid

    def clear_hash(self, bid: int) -> None:
        blk = self.blocks[bid]
        if blk.hash is not None and self.hash_to_block.get(blk.hash) == bid:
            del self.hash_to_block[blk.hash]
        blk.hash, blk.token_ids = None, ()


class CpuBlockPool:
    """Swap pages in pinned host memory; ``allocate_many`` is all-or-nothing."""

    def __init__(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        self.free: deque[int] = deque(range(num_blocks))
        self.saved_hash: dict[int, tuple[int, tuple[int, ...]]] = {}

    @property
    def num_free(self) -> int:
        return len(self.free)

    def allocate_many(self, n: int) -> list[int]:
        if n > len(self.free):
            raise OutOfBlocks(f"need {n} CPU pages, {len(self.free)} free")
        return [self.free.popleft() for _ in range(n)]

    def release(self, bid: int) -> None:
        self.saved_hash.pop(bid, None)
        self.free.append(bid)
