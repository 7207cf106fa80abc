"""Page-table orchestration and the two prefix caches.

* Text prompts: chained content hashes over full pages let identical prefixes share pages
  (never for multimodal prompts, whose placeholder tokens say nothing about the pixels).
* Multimodal prompts: the question-independent prefix (everything up to the last visual
  placeholder) is cached per ``media_key`` as a list of read-only pages plus the
  logical-to-physical layout left by compaction.  A later request with the same media
  borrows the full pages, gets a private copy of the partial tail page (a ``copy_prefix``
  transfer) and only computes its own question.  Entries may occupy any free page of the
  pool and are evicted on demand, lowest ``benefit_tokens * (1 + hits) / resident_pages``
  first.
* Copy-on-write, append, swap-out / swap-in (hashes, scales and layouts survive) and the
  plan / commit halves of physical compaction.

Behavioural reference: ``prism_infer/engine/block_manager.py:51-937`` and
``prism_infer/engine/kv_compaction_coordinator.py:27-175``.
"""

from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass
from typing import Sequence as Seq

from .block_pool import CpuBlockPool, GpuBlockPool, OutOfBlocks
from .contracts import KVTransferPlan
from .kv_layout import CompactionPlan, KVLayout
from .sequence import Sequence
from ..observability import emit_kv_event


def chain_hash(token_ids: Seq[int], prefix: int | None) -> int:
    h = hashlib.blake2b(digest_size=8)
    if prefix is not None:
        h.update(struct.pack("<Q", prefix & 0xFFFFFFFFFFFFFFFF))
    h.update(struct.pack(f"<{len(token_ids)}q", *token_ids))
    return int.from_bytes(h.digest(), "little")


def multimodal_prefix_id(media_key: str, tokens: Seq[int]) -> str:
    digest = hashlib.sha256(struct.pack(f"<{len(tokens)}q", *tokens)).hexdigest()
    return f"{media_key}:{len(tokens)}:{digest}"


@dataclass
class PrefixEntry:
    cache_id: str
    check: int                      # independent digest of the prefix tokens (collision check)
    prefix_len: int                 # logical tokens covered
    pages: list[int]                # full pages, then the tail clone (if tail_rows > 0)
    tail_rows: int
    layout: KVLayout | None
    hits: int = 0
    last_use: int = 0

    @property
    def physical_len(self) -> int:
        return self.layout.physical_prefix_len if self.layout is not None else self.prefix_len

    @property
    def dropped(self) -> int:
        return self.layout.dropped if self.layout is not None else 0

    def score(self) -> float:
        return self.prefix_len * (1 + self.hits) / max(1, len(self.pages))


@dataclass
class PrefixCacheCounters:
    probes: int = 0
    probe_hits: int = 0
    stale_probes: int = 0
    hits: int = 0
    misses: int = 0
    stores: int = 0
    store_skipped: int = 0
    evictions: int = 0
    collisions: int = 0
    tail_clones: int = 0
    tokens_reused: int = 0
    pages_shared: int = 0

    def snapshot(self) -> dict[str, int]:
        return dict(self.__dict__)


class BlockManager:
    def __init__(self, num_gpu_blocks: int, page: int, num_cpu_blocks: int = 0, *, enable_prefix_caching: bool = True) -> None:
        self.page = page
        self.gpu = GpuBlockPool(num_gpu_blocks)
        self.cpu = CpuBlockPool(num_cpu_blocks)
        self.enable_prefix_caching = enable_prefix_caching
        self.entries: dict[str, PrefixEntry] = {}
        self.counters = PrefixCacheCounters()
        self._clock = 0
        self._entry_pages: set[int] = set()   # pages held by some prefix entry
        self._evictable = 0                   # of those, pages no sequence borrows
        Sequence.block_size = page

    # ------------------------------------------------------------------ capacity
    # A page held by a prefix entry can be reclaimed when the entry is its only holder.  The count
    # of such pages is kept up to date where reference counts of entry pages change (store, hit,
    # release of a borrower, eviction), because ``can_append`` asks for it once per sequence
    # and decode step.
    def _retain(self, page: int) -> None:
        if page in self._entry_pages and self.gpu.blocks[page].ref_count == 1:
            self._evictable -= 1
        self.gpu.retain(page)

    def _release(self, page: int) -> None:
        self.gpu.release(page)
        if page in self._entry_pages and self.gpu.blocks[page].ref_count == 1:
            self._evictable += 1

    def _evictable_pages(self) -> int:
        return self._evictable

    def _freed_by_eviction(self, entry: PrefixEntry) -> int:
        return sum(1 for p in entry.pages if self.gpu.blocks[p].ref_count == 1)

    def _ensure_free(self, n: int, protect: str | None = None) -> bool:
        """Evict prefix entries, lowest score first, until ``n`` pages are free.  An entry whose
        pages are all still borrowed by running sequences would free nothing: it stays."""
        while self.gpu.num_free < n:
            victims = [e for e in self.entries.values() if e.cache_id != protect and self._freed_by_eviction(e) > 0]
            if not victims:
                return False
            victim = min(victims, key=lambda e: (e.score(), e.last_use))
            self._evict(victim)
        return True

    def _evict(self, entry: PrefixEntry) -> None:
        freed = 0
        for p in entry.pages:
            if self.gpu.blocks[p].ref_count == 1:
                self._evictable -= 1
                freed += 1
            self._entry_pages.discard(p)
            self.gpu.release(p)
        del self.entries[entry.cache_id]
        self.counters.evictions += 1
        emit_kv_event("evict", cache_id=entry.cache_id, pages=len(entry.pages), freed=freed, hits=entry.hits)

    def num_free_with_eviction(self) -> int:
        return self.gpu.num_free + self._evictable_pages()

    # -------------------------------------------------------------- multimodal prefix
    def _prefix_identity(self, seq: Sequence) -> tuple[str, int, int] | None:
        if not self.enable_prefix_caching or seq.multimodal_prefix_cache_key is None:
            return None
        boundary = seq.multimodal_prefix_boundary
        if boundary <= 0 or boundary >= seq.num_prompt_tokens:
            return None
        toks = seq.token_ids[:boundary]
        return multimodal_prefix_id(seq.multimodal_prefix_cache_key, toks), chain_hash(toks, None), boundary

    def probe_multimodal_prefix(self, seq: Sequence) -> PrefixEntry | None:
        ident = self._prefix_identity(seq)
        if ident is None:
            return None
        self.counters.probes += 1
        entry = self.entries.get(ident[0])
        if entry is None:
            return None
        if entry.check != ident[1] or entry.prefix_len != ident[2]:
            self.counters.collisions += 1
            return None
        self.counters.probe_hits += 1
        return entry

    def _pages_for_hit(self, seq: Sequence, entry: PrefixEntry) -> int:
        total = -(-(len(seq) - entry.dropped) // self.page)
        return total - (len(entry.pages) - (1 if entry.tail_rows else 0))

    # --------------------------------------------------------------------- allocate
    def can_allocate(self, seq: Sequence) -> bool:
        entry = self.probe_multimodal_prefix(seq) if seq.is_multimodal else None
        need = self._pages_for_hit(seq, entry) if entry is not None else seq.blocks_needed(len(seq))
        return self.num_free_with_eviction() >= need

    def allocate(self, seq: Sequence, *, expected_hit: bool | None = None) -> KVTransferPlan:
        """Give ``seq`` pages for its whole prompt; returns the copies that must run first."""
        if seq.block_table:
            raise RuntimeError(f"sequence {seq.seq_id} already owns pages")
        if seq.is_multimodal:
            entry = self.probe_multimodal_prefix(seq)
            if entry is None and expected_hit:
                self.counters.stale_probes += 1
            if entry is not None:
                plan = self._allocate_prefix_hit(seq, entry)
                if plan is not None:
                    return plan
            if self._prefix_identity(seq) is not None:
                self.counters.misses += 1
            self._allocate_dense(seq, share=False)
            return KVTransferPlan()
        self._allocate_dense(seq, share=self.enable_prefix_caching)
        return KVTransferPlan()

    def _allocate_prefix_hit(self, seq: Sequence, entry: PrefixEntry) -> KVTransferPlan | None:
        fresh_needed = self._pages_for_hit(seq, entry)
        if not self._ensure_free(fresh_needed, protect=entry.cache_id):
            return None
        n_full = len(entry.pages) - (1 if entry.tail_rows else 0)
        table: list[int] = []
        try:
            for p in entry.pages[:n_full]:
                self._retain(p)
                table.append(p)
            fresh = self.gpu.allocate_many(fresh_needed)
        except OutOfBlocks:
            for p in table:
                self._release(p)
            return None
        table.extend(fresh)
        copies: tuple[tuple[int, int, int], ...] = ()
        if entry.tail_rows:
            copies = ((entry.pages[-1], fresh[0], entry.tail_rows),)
            self.counters.tail_clones += 1
        seq.block_table = table
        seq.block_table_version += 1
        seq.kv_layout = entry.layout
        seq.num_computed_tokens = seq.num_cached_tokens = entry.prefix_len
        self._clock += 1
        entry.hits += 1
        entry.last_use = self._clock
        self.counters.hits += 1
        self.counters.tokens_reused += entry.prefix_len
        self.counters.pages_shared += n_full
        emit_kv_event("prefix_hit", seq_id=seq.seq_id, cache_id=entry.cache_id, tokens=entry.prefix_len, shared_pages=n_full,
                      fresh_pages=len(fresh), tail_rows=entry.tail_rows)
        return KVTransferPlan(copy_prefix=copies)

    def _allocate_dense(self, seq: Sequence, *, share: bool) -> None:
        n_pages = seq.blocks_needed(len(seq))
        table: list[int] = []
        pending: list[tuple[int, int, tuple[int, ...]]] = []
        cached_tokens = 0
        h: int | None = None
        still_hitting = share
        try:
            for i in range(n_pages):
                toks = tuple(seq.token_ids[i * self.page:(i + 1) * self.page])
                full = len(toks) == self.page
                h = chain_hash(toks, h) if (share and full) else None
                bid = self.gpu.lookup(h, toks) if (still_hitting and h is not None) else None
                # the last prompt token must be computed to produce logits
                if bid is not None and (i + 1) * self.page >= len(seq):
                    bid = None
                if bid is not None:
                    self._retain(bid)
                    cached_tokens += self.page
                else:
                    still_hitting = False
                    if not self._ensure_free(1):
                        raise OutOfBlocks("no free GPU page")
                    bid = self.gpu.allocate()
                    if h is not None:
                        # the page holds no KV yet: its hash becomes visible to other requests
                        # only after the chunk that fills it has run (publish_computed_pages)
                        pending.append((i, h, toks))
                table.append(bid)
        except OutOfBlocks:
            for p in table:
                self._release(p)
            raise
        emit_kv_event("allocate", seq_id=seq.seq_id, pages=len(table), cached_tokens=cached_tokens)
        seq.block_table = table
        seq.block_table_version += 1
        seq.kv_layout = None
        seq.num_cached_tokens = cached_tokens
        seq.num_computed_tokens = cached_tokens
        seq.unpublished_hashes = pending

    def publish_computed_pages(self, seq: Sequence) -> int:
        """Publish the content hashes of ``seq``'s own prompt pages that are now fully computed
        (every token of the page is below ``num_computed_tokens``).  Called after each prefill
        step; a page that another request published first keeps that request's copy.  Pages of a
        sequence that is cancelled or preempted before they are computed are never published, so a
        later identical prompt cannot be served from rows nobody wrote."""
        if not seq.unpublished_hashes or seq.kv_layout is not None:
            return 0
        done, rest = 0, []
        for i, h, toks in seq.unpublished_hashes:
            if (i + 1) * self.page <= seq.num_computed_tokens and i < len(seq.block_table):
                if self.gpu.lookup(h, toks) is None:
                    self.gpu.publish(seq.block_table[i], h, toks)
                done += 1
            else:
                rest.append((i, h, toks))
        seq.unpublished_hashes = rest
        return done

    def deallocate(self, seq: Sequence) -> None:
        seq.unpublished_hashes = []
        for p in reversed(seq.block_table):
            self._release(p)
        if seq.block_table:
            emit_kv_event("free", seq_id=seq.seq_id, pages=len(seq.block_table))
        seq.block_table = []
        seq.block_table_version += 1
        for p in seq.cpu_block_table:
            self.cpu.release(p)
        seq.cpu_block_table = []
        seq.num_computed_tokens = 0
        seq.kv_layout = None

    # ------------------------------------------------------------- decode-time growth
    def needs_new_page(self, seq: Sequence) -> bool:
        """True when the next token's KV row opens a new page."""
        return seq.physical_len() > len(seq.block_table) * self.page

    def can_append(self, seq: Sequence) -> bool:
        need = 1 if self.needs_new_page(seq) else 0
        if not need and seq.block_table and self.gpu.blocks[seq.block_table[-1]].ref_count > 1:
            need = 1  # copy-on-write of a shared tail
        return need == 0 or self.num_free_with_eviction() >= need

    def append(self, seq: Sequence) -> tuple[tuple[int, int], ...]:
        """Make room for the KV row of ``seq``'s last token; returns copy-on-write pairs."""
        cow: list[tuple[int, int]] = []
        if self.needs_new_page(seq):
            if not self._ensure_free(1):
                raise OutOfBlocks("no free GPU page for decode")
            seq.block_table.append(self.gpu.allocate())
            seq.block_table_version += 1
        else:
            last = seq.block_table[-1]
            if self.gpu.blocks[last].ref_count > 1:
                pair = self.copy_on_write(seq, len(seq.block_table) - 1)
                if pair is not None:
                    cow.append(pair)
        return tuple(cow)

    def copy_on_write(self, seq: Sequence, index: int) -> tuple[int, int] | None:
        old = seq.block_table[index]
        if self.gpu.blocks[old].ref_count <= 1:
            return None
        if not self._ensure_free(1):
            raise OutOfBlocks("no free GPU page for copy-on-write")
        new = self.gpu.allocate()
        self._release(old)
        emit_kv_event("copy_on_write", seq_id=seq.seq_id, src=old, dst=new)
        seq.block_table[index] = new
        seq.block_table_version += 1
        return old, new

    # ------------------------------------------------------------------------- swap
    def can_swap_out(self, seq: Sequence) -> bool:
        return self.cpu.num_free >= len(seq.block_table)

    def swap_out(self, seq: Sequence) -> tuple[tuple[int, int], ...]:
        cpu_pages = self.cpu.allocate_many(len(seq.block_table))
        pairs = []
        for g, c in zip(seq.block_table, cpu_pages):
            blk = self.gpu.blocks[g]
            if blk.hash is not None:
                self.cpu.saved_hash[c] = (blk.hash, blk.token_ids)
            pairs.append((g, c))
            self._release(g)
        emit_kv_event("swap_out", seq_id=seq.seq_id, pages=len(pairs))
        seq.cpu_block_table = cpu_pages
        seq.block_table = []
        seq.block_table_version += 1
        return tuple(pairs)

    def can_swap_in(self, seq: Sequence) -> bool:
        return self.num_free_with_eviction() >= len(seq.cpu_block_table)

    def swap_in(self, seq: Sequence) -> tuple[tuple[int, int], ...]:
        n = len(seq.cpu_block_table)
        if not self._ensure_free(n):
            raise OutOfBlocks("no free GPU pages to swap in")
        gpu_pages = self.gpu.allocate_many(n)
        pairs = []
        for c, g in zip(seq.cpu_block_table, gpu_pages):
            saved = self.cpu.saved_hash.get(c)
            if saved is not None and self.gpu.lookup(saved[0], saved[1]) is None:
                self.gpu.publish(g, saved[0], saved[1])
            pairs.append((c, g))
            self.cpu.release(c)
        emit_kv_event("swap_in", seq_id=seq.seq_id, pages=len(pairs))
        seq.block_table = gpu_pages
        seq.cpu_block_table = []
        seq.block_table_version += 1
        return tuple(pairs)

    # ------------------------------------------------------------------- compaction
    def build_compaction_plan(self, seq: Sequence, retained_positions: Seq[int], prefix_len: int) -> CompactionPlan | None:
        """Plan moving the retained rows of ``[0, prefix_len)`` to the front of ``seq``'s own
        pages.  Returns ``None`` when nothing would be dropped."""
        if seq.kv_layout is not None:
            raise RuntimeError("sequence is already compacted")
        if seq.num_computed_tokens < prefix_len:
            raise RuntimeError("compaction must run after the prefix has been computed")
        if any(self.gpu.blocks[p].ref_count > 1 for p in seq.block_table):
            raise RuntimeError("cannot compact shared pages")
        layout = KVLayout(prefix_len, tuple(retained_positions))
        if layout.dropped == 0:
            return None
        page, table = self.page, seq.block_table
        # rows computed behind the prefix (a prompt prefilled in one piece) move down with it
        moved = tuple(layout.retained_positions) + tuple(range(prefix_len, seq.num_computed_tokens))
        src = tuple(table[p // page] * page + p % page for p in moved)
        dst = tuple(table[i // page] * page + i % page for i in range(len(moved)))
        need = -(-(len(seq) - layout.dropped) // page)
        return CompactionPlan(seq.seq_id, layout, src, dst, tuple(table[:need]), tuple(table[need:]), seq.block_table_version)

    def commit_compaction(self, seq: Sequence, plan: CompactionPlan) -> None:
        """Install the layout after the device copy finished; refuses stale plans."""
        if plan.seq_id != seq.seq_id or plan.block_table_version != seq.block_table_version:
            raise RuntimeError("stale compaction plan")
        for p in seq.block_table:
            self.gpu.clear_hash(p)
        seq.unpublished_hashes = []
        for p in plan.released_blocks:
            self._release(p)
        seq.block_table = list(plan.kept_blocks)
        seq.block_table_version += 1
        seq.kv_layout = plan.layout

    # ------------------------------------------------------------------ prefix store
    def store_multimodal_prefix(self, seq: Sequence) -> tuple[tuple[int, int, int], ...]:
        """Publish ``seq``'s computed multimodal prefix; returns the tail-clone copy to run."""
        ident = self._prefix_identity(seq)
        if ident is None or ident[0] in self.entries:
            return ()
        cache_id, check, boundary = ident
        if seq.num_computed_tokens < boundary:
            return ()
        layout = seq.kv_layout
        if layout is not None and layout.logical_prefix_len != boundary:
            return ()
        phys = layout.physical_prefix_len if layout is not None else boundary
        n_full, tail_rows = phys // self.page, phys % self.page
        pages = list(seq.block_table[:n_full])
        copies: tuple[tuple[int, int, int], ...] = ()
        if tail_rows:
            if self.gpu.num_free < 1:
                self.counters.store_skipped += 1
                return ()
            clone = self.gpu.allocate()
            copies = ((seq.block_table[n_full], clone, tail_rows),)
        for p in pages:
            self.gpu.retain(p)
        if tail_rows:
            pages.append(clone)
        for p in pages:
            self._entry_pages.add(p)
            if self.gpu.blocks[p].ref_count == 1:  # the tail clone; borrowed pages count once their sequence lets go
                self._evictable += 1
        self._clock += 1
        self.entries[cache_id] = PrefixEntry(cache_id, check, boundary, pages, tail_rows, layout, 0, self._clock)
        self.counters.stores += 1
        emit_kv_event("prefix_store", seq_id=seq.seq_id, cache_id=cache_id, tokens=boundary, pages=len(pages), tail_rows=tail_rows)
        return copies

    # --------------------------------------------------------------------- metadata
    def prefix_cache_metadata(self) -> dict[str, object]:
        resident = sum(len(e.pages) for e in self.entries.values())
        return {
            "enabled": self.enable_prefix_caching,
            "entries": len(self.entries),
            "resident_pages": resident,
            "resident_tokens": sum(e.physical_len for e in self.entries.values()),
            "logical_tokens": sum(e.prefix_len for e in self.entries.values()),
            "free_pages": self.gpu.num_free,
            "total_pages": self.gpu.num_blocks,
            **self.counters.snapshot(),
        }
