"""Continuous-batching scheduler (host only, no CUDA).

Queues: waiting, running (prefilling or decoding), swapped, plus ledgers of rejected and
cancelled requests.  Each call to ``schedule`` returns one immutable ``BatchPlan``:

* a prefill plan continues partially prefilled running sequences first, then admits
  waiting sequences under the token, sequence and vision-patch budgets;
* a decode plan swaps sequences back in, makes room for one more KV row per sequence
  (copy-on-write if the tail page is shared) and preempts last-in-first-out when pages run
  out: swap to CPU pages when the pool has room, otherwise drop the KV and recompute.

``postprocess`` appends sampled tokens and finishes sequences on EOS or length.
Behavioural reference: ``prism_infer/engine/scheduler.py:91-761``.
"""

from __future__ import annotations

import time
from collections import deque
from typing import Callable, Iterable

from .block_manager import BlockManager
from .block_pool import OutOfBlocks
from .contracts import BatchPlan, KVTransferPlan, Phase, PrefillSlice, RequestOutput
from .request import RequestState
from .scheduler_policy import FCFSPolicy, make_policy
from .sequence import Sequence


class Scheduler:
    def __init__(self, config, block_manager: BlockManager | None = None, *, policy: FCFSPolicy | None = None,
                 metrics=None, clock_ns: Callable[[], int] = time.perf_counter_ns) -> None:
        self.config = config
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.max_vision_patches = config.max_vision_patches_per_batch
        self.max_model_len = config.max_model_len
        self.eos = config.eos
        self.block_manager = block_manager or BlockManager(
            config.num_kvcache_blocks, config.kvcache_block_size, config.num_cpu_blocks,
            enable_prefix_caching=config.enable_prefix_caching)
        self.policy = policy or make_policy(config)
        self.metrics = metrics
        self.clock_ns = clock_ns
        # a chunk must end on the multimodal prefix boundary only where the prefix is compacted in
        # place before the rest of the prompt is written behind it; a dense prefix is published
        # from whichever chunk crosses the boundary, without an extra prefill step
        self.stop_at_prefix = bool(config.compacts_visual_tokens)
        # attention strategy: a prompt that fits one chunk is prefilled whole (its last query scores the
        # visual tokens); longer prompts still end a chunk on the boundary and compact uniformly
        self.whole_prompt_first = bool(config.compacts_visual_tokens and getattr(config, "visual_pruning_strategy", "uniform") == "attention")
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.swapped: deque[Sequence] = deque()
        self.rejected: list[Sequence] = []
        self.cancelled: list[Sequence] = []
        self.consecutive_prefill_batches = 0
        self.counters = {
            "admitted": 0, "rejected": 0, "cancelled": 0, "finished": 0, "preempt_swap": 0, "preempt_recompute": 0,
            "swap_in": 0, "prefill_batches": 0, "decode_batches": 0, "peak_running": 0, "peak_waiting": 0,
            "peak_swapped": 0,
        }

    # ----------------------------------------------------------------------- queues
    def add(self, seq: Sequence) -> bool:
        """Admit to the waiting queue or reject; returns True when admitted."""
        verdict = self.policy.admit(seq, len(self.waiting))
        if not verdict.ok:
            seq.lifecycle.transition(RequestState.REJECTED, verdict.reason)
            self.rejected.append(seq)
            self.counters["rejected"] += 1
            return False
        self.waiting.append(seq)
        self.counters["admitted"] += 1
        self.counters["peak_waiting"] = max(self.counters["peak_waiting"], len(self.waiting))
        return True

    def is_finished(self) -> bool:
        return not (self.waiting or self.running or self.swapped)

    @property
    def num_decoding(self) -> int:
        return sum(1 for s in self.running if s.state is RequestState.DECODING)

    def find(self, seq_id: int) -> Sequence | None:
        for q in (self.running, self.waiting, self.swapped):
            for s in q:
                if s.seq_id == seq_id:
                    return s
        return None

    # --------------------------------------------------------------------- schedule
    def schedule(self) -> BatchPlan:
        prefilling = [s for s in self.running if s.state is RequestState.PREFILLING]
        can_decode = self.num_decoding > 0 or bool(self.swapped)
        if prefilling or self.waiting:
            self._order_waiting()
            head = prefilling[0] if prefilling else (self.waiting[0] if self.waiting else None)
            if not can_decode or self.policy.allow_prefill(self, head):
                plan = self._prefill_plan(prefilling)
                if plan is not None:
                    self.consecutive_prefill_batches += 1
                    self.counters["prefill_batches"] += 1
                    self.policy.on_prefill_batch(plan.seqs)
                    return plan
        if can_decode:
            plan = self._decode_plan()
            if plan is not None:
                self.consecutive_prefill_batches = 0
                self.counters["decode_batches"] += 1
                self.policy.on_decode_batch()
                return plan
        if prefilling or self.waiting:  # policy held prefill back but nothing can decode
            plan = self._prefill_plan(prefilling)
            if plan is not None:
                self.counters["prefill_batches"] += 1
                return plan
        return BatchPlan(Phase.IDLE)

    def _order_waiting(self) -> None:
        items = list(self.waiting)
        self.policy.order_waiting(items, self.clock_ns())
        self.waiting = deque(items)

    def schedule_prefill(self, *, max_cost_tier: int | None = None) -> BatchPlan | None:
        """A prefill plan now.  With ``max_cost_tier`` (SLO-aware policy) only waiting requests of that cost tier or
        a cheaper one are admitted and nothing that is already prefilling is continued: the plan that interrupts a
        pending, more expensive prefill."""
        if max_cost_tier is None:
            return self._prefill_plan([s for s in self.running if s.state is RequestState.PREFILLING])
        tier = getattr(self.policy, "cost_tier", None)
        if tier is None:
            return None
        self._order_waiting()
        items = list(self.waiting)  # eligible requests first, both groups in policy order
        self.waiting = deque([s for s in items if tier(s) <= max_cost_tier] + [s for s in items if tier(s) > max_cost_tier])
        plan = self._prefill_plan([], max_cost_tier=max_cost_tier)
        self._order_waiting()
        if plan is not None:
            self.counters["prefill_batches"] += 1
            self.policy.on_prefill_batch(plan.seqs)
        return plan

    def schedule_decode(self, *, count: bool = False) -> BatchPlan | None:
        """A decode plan of the running sequences, whatever waits.  With ``count`` the plan is booked the way
        ``schedule`` books its own decode batches (prefill / decode alternation, heavy-prefill spacing, counters)."""
        plan = self._decode_plan()
        if plan is not None and count and plan.phase is Phase.DECODE:
            self.consecutive_prefill_batches = 0
            self.counters["decode_batches"] += 1
            self.policy.on_decode_batch()
        return plan

    def _prefill_plan(self, prefilling: list[Sequence], *, max_cost_tier: int | None = None) -> BatchPlan | None:
        budget = self.max_num_batched_tokens
        patches_left = self.max_vision_patches
        seqs: list[Sequence] = []
        slices: list[PrefillSlice] = []
        copies: list[tuple[int, int, int]] = []
        patches = 0

        def try_add(seq: Sequence) -> bool:
            nonlocal budget, patches_left, patches
            stop = self.stop_at_prefix
            if stop and self.whole_prompt_first and seq.num_computed_tokens == 0 and seq.num_cached_tokens == 0:
                limit = min(budget, self.policy.max_chunk) if self.policy.chunked else budget
                stop = len(seq) > limit
            n = self.policy.prefill_token_count(seq, budget, stop_at_prefix=stop)
            if n <= 0:
                return False
            start = seq.num_computed_tokens
            p = seq.vision_patch_count(start, start + n)
            if p > patches_left and seqs:
                return False
            seqs.append(seq)
            slices.append(PrefillSlice(start, n))
            budget -= n
            patches_left -= p
            patches += p
            return True

        for seq in prefilling:
            if budget <= 0:
                break
            try_add(seq)
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            if max_cost_tier is not None and self.policy.cost_tier(seq) > max_cost_tier:
                break
            if not self.policy.may_admit(self, seq) or not self.block_manager.can_allocate(seq):
                break
            try:
                transfers = self.block_manager.allocate(seq)
            except OutOfBlocks:
                break
            self.waiting.popleft()
            copies.extend(transfers.copy_prefix)
            seq.lifecycle.transition(RequestState.PREFILLING, "admitted")
            self.running.append(seq)
            if self.metrics is not None:
                self.metrics.on_request_scheduled(seq)
            try_add(seq)
        self.counters["peak_running"] = max(self.counters["peak_running"], len(self.running))
        if not seqs:
            return None
        return BatchPlan(Phase.PREFILL, tuple(seqs), tuple(slices), KVTransferPlan(copy_prefix=tuple(copies)),
                         sum(s.length for s in slices), patches)

    def _decode_plan(self) -> BatchPlan | None:
        bm = self.block_manager
        swap_in: list[tuple[int, int]] = []
        swap_out: list[tuple[int, int]] = []
        cow: list[tuple[int, int]] = []
        while self.swapped and len(self.running) < self.max_num_seqs and bm.can_swap_in(self.swapped[0]):
            seq = self.swapped.popleft()
            swap_in.extend(bm.swap_in(seq))
            seq.lifecycle.transition(RequestState.DECODING, "swap_in")
            self.running.append(seq)
            self.counters["swap_in"] += 1
        batch: list[Sequence] = []
        preempted = False  # membership in ``running`` only changes through a preemption in this pass
        for seq in list(self.running):
            if seq.state is not RequestState.DECODING or (preempted and seq not in self.running):
                continue
            while not bm.can_append(seq):
                victim = self.policy.pick_victim([s for s in self.running if s.state is RequestState.DECODING])
                swap_out.extend(self.preempt(victim))
                preempted = True
                if victim is seq:
                    break
            if preempted and (seq.state is not RequestState.DECODING or seq not in self.running):
                continue
            cow.extend(bm.append(seq))
            batch.append(seq)
            if len(batch) >= self.max_num_seqs:
                break
        if preempted:
            batch = [s for s in batch if s in self.running and s.state is RequestState.DECODING]
        if not batch:
            if swap_out:
                return BatchPlan(Phase.IDLE, kv_transfers=KVTransferPlan(swap_out=tuple(swap_out)))
            return None
        return BatchPlan(Phase.DECODE, tuple(batch), (), KVTransferPlan(copy_on_write=tuple(cow), swap_out=tuple(swap_out),
                                                                          swap_in=tuple(swap_in)), len(batch), 0)

    # ---------------------------------------------------------------------- preempt
    def preempt(self, seq: Sequence) -> tuple[tuple[int, int], ...]:
        """Free ``seq``'s GPU pages: swap to CPU pages if possible, else recompute later."""
        self.running.remove(seq)
        bm = self.block_manager
        if seq.state is RequestState.DECODING and bm.can_swap_out(seq) and bm.cpu.num_blocks > 0:
            pairs = bm.swap_out(seq)
            seq.lifecycle.transition(RequestState.SWAPPED, "preempt_swap")
            self.swapped.append(seq)
            self.counters["preempt_swap"] += 1
            self.counters["peak_swapped"] = max(self.counters["peak_swapped"], len(self.swapped))
            return pairs
        bm.deallocate(seq)
        seq.num_cached_tokens = 0
        seq.lifecycle.transition(RequestState.WAITING, "preempt_recompute")
        self.waiting.appendleft(seq)
        self.counters["preempt_recompute"] += 1
        return ()

    # ------------------------------------------------------------------ postprocess
    def postprocess(self, plan: BatchPlan, tokens: Iterable[int | None]) -> list[RequestOutput]:
        outputs: list[RequestOutput] = []
        for i, (seq, tok) in enumerate(zip(plan.seqs, tokens)):
            if seq.is_finished:  # cancelled while the step was in flight
                continue
            if plan.phase is Phase.PREFILL:
                seq.num_computed_tokens += plan.slices[i].length
                self.block_manager.publish_computed_pages(seq)
                if seq.num_computed_tokens < len(seq) or tok is None:
                    outputs.append(RequestOutput(seq.seq_id, None, False))
                    continue
                seq.lifecycle.transition(RequestState.DECODING, "prefill_done")
            else:
                seq.num_computed_tokens += 1
            seq.append_token(int(tok))
            if self.metrics is not None:
                self.metrics.on_tokens(seq, 1)
            reason = None
            if not seq.ignore_eos and int(tok) == self.eos:
                reason = "eos"
            elif seq.num_completion_tokens >= seq.max_tokens:
                reason = "length"
            elif len(seq) >= self.max_model_len:
                reason = "length"
            if reason is not None:
                self._finish(seq, reason)
            outputs.append(RequestOutput(seq.seq_id, int(tok), reason is not None, reason,
                                         tuple(seq.completion_token_ids) if reason else ()))
        return outputs

    def _finish(self, seq: Sequence, reason: str) -> None:
        seq.lifecycle.transition(RequestState.FINISHED, reason)
        self.block_manager.deallocate(seq)
        if seq in self.running:
            self.running.remove(seq)
        self.counters["finished"] += 1
        if self.metrics is not None:
            self.metrics.on_request_finished(seq)

    # ----------------------------------------------------------------------- cancel
    def cancel(self, seq_id: int, reason: str = "cancelled") -> bool:
        seq = self.find(seq_id)
        if seq is None:
            return False
        for q in (self.running, self.waiting, self.swapped):
            if seq in q:
                q.remove(seq)
        self.block_manager.deallocate(seq)
        seq.lifecycle.transition(RequestState.CANCELLED, reason)
        self.cancelled.append(seq)
        self.counters["cancelled"] += 1
        if self.metrics is not None:
            self.metrics.on_request_finished(seq)
        return True

    def metrics_snapshot(self) -> dict[str, object]:
        return {
            **self.counters, "waiting": len(self.waiting), "running": len(self.running), "swapped": len(self.swapped),
            "free_gpu_pages": self.block_manager.gpu.num_free, "free_cpu_pages": self.block_manager.cpu.num_free,
        }
