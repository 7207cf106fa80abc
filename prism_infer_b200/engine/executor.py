"""Applies one ``BatchPlan`` (reference ``prism_infer/engine/executor.py:27-209``).

Order inside a step: page transfers (prefix-row copies, copy-on-write, swap-out,
swap-in), model execution on every rank, then for prefill sequences that just reached
their multimodal prefix boundary: visual-token compaction (plan, device copy, commit) and
publication of the prefix to the cache (which may add a tail-clone copy).  Every device
action goes through ``runner.call`` so tensor-parallel ranks stay in lock step.
"""

from __future__ import annotations

import collections
import time

from .block_manager import BlockManager
from .contracts import BatchPlan, ExecutionResult, KVTransferPlan, Phase
from .input_preparation import ModelInputPreparer
from .visual_pruning import PruningConfig, compute_pruning_decision, retained_positions
from ..observability import emit_kv_event, profile_region


class LocalRunnerGroup:
    """Single-rank dispatch: direct method calls on the in-process runner."""

    def __init__(self, runner) -> None:
        self.runner = runner

    def call(self, method: str, *args):
        return getattr(self.runner, method)(*args)

    def close(self) -> None:
        self.runner.exit()


class ModelExecutor:
    def __init__(self, config, runners, block_manager: BlockManager) -> None:
        self.config = config
        self.runners = runners
        self.bm = block_manager
        self.preparer = ModelInputPreparer(config.kvcache_block_size, -(-config.max_model_len // config.kvcache_block_size))
        self.compact = config.compacts_visual_tokens
        self.pruning = PruningConfig(config.visual_pruning_keep_ratio, config.visual_pruning_min_keep_tokens,
                                     config.visual_pruning_video_min_keep_tokens,
                                     "uniform" if config.visual_pruning_strategy == "attention" else config.visual_pruning_strategy)
        self._have_visual: set[int] = set()
        # attention strategy: prompts prefilled in one piece are scored by the last query's attention
        # over their visual tokens (last N decoder layers) and compacted by those scores; prompts
        # that need several chunks fall back to the uniform selection at the prefix boundary
        self.attention_strategy = bool(self.compact and config.visual_pruning_strategy == "attention")
        n_layers = config.arch.text.num_layers
        last_n = max(1, min(n_layers, int(config.visual_pruning_attention_last_n_layers)))
        self.score_layers = list(range(n_layers - last_n, n_layers))
        self.pruning_scored = PruningConfig(config.visual_pruning_keep_ratio, config.visual_pruning_min_keep_tokens,
                                            config.visual_pruning_video_min_keep_tokens, "attention")
        self.attention_counters = {"scored": 0, "uniform_fallback": 0}
        # what was (or, in shadow mode, would have been) kept of every prompt's visual tokens; bounded for a long-running server
        self.shadow = bool(getattr(config, "enable_visual_pruning_shadow", False)) and not self.compact
        self.pruning_decisions: collections.deque[dict] = collections.deque(maxlen=4096)

    def _record_decision(self, seq, decision, *, applied: bool) -> None:
        """One ledger entry per prompt (reference ``engine/compression.py:335-470`` builds the same record per batch)."""
        self.pruning_decisions.append({
            "seq_id": seq.seq_id, "applied": applied, "strategy": decision.strategy, "total_visual_tokens": decision.total_visual_tokens,
            "kept": len(decision.kept), "dropped": len(decision.dropped), "keep_ratio_actual": decision.keep_ratio_actual,
            "spans": [{"modality": sp.modality, "start": sp.start, "end": sp.end} for sp in decision.spans],
            "prefix_len": int(seq.multimodal_prefix_boundary)})

    def mark_visual_ready(self, seq_id: int) -> None:
        """The runner already holds this sequence's vision result (hydrated at submission)."""
        self._have_visual.add(seq_id)

    def drop_visual(self, seq_id: int) -> None:
        """A sequence left before its prefill consumed the vision result: free it on the ranks."""
        if seq_id in self._have_visual:
            self._have_visual.discard(seq_id)
            self.runners.call("release_visual", seq_id)

    def hydrate_vision(self, plan: BatchPlan) -> int:
        """Cooperative prefill quantum: push the plan's pending vision-tower work through the
        runner now (page transfers included) and leave the language prefill to a later step,
        so running decodes are not stalled behind vision + prefill in one piece (reference
        ``engine/llm_engine.py:913-1017``).  Returns the number of sequences hydrated."""
        if not plan.kv_transfers.empty:
            self.runners.call("apply_kv_transfers", plan.kv_transfers)
        inputs = self.preparer.prepare(plan, self._have_visual)
        for job in inputs.vision_jobs:
            self.runners.call("encode_for_sequence", job)
            self._have_visual.add(job.seq_id)
        return len(inputs.vision_jobs)

    def begin_hydrate(self, plan: BatchPlan) -> dict | None:
        """``hydrate_vision`` in block quanta: page transfers and input preparation now, the vision tower of each
        pending job a few blocks at a time through ``advance_hydrate``.  None when the plan has no tower work."""
        if not plan.kv_transfers.empty:
            self.runners.call("apply_kv_transfers", plan.kv_transfers)
        inputs = self.preparer.prepare(plan, self._have_visual)
        if not inputs.vision_jobs:
            return None
        return {"jobs": list(inputs.vision_jobs), "next": 0, "encode": None, "quanta": 0}

    def advance_hydrate(self, handle: dict, max_blocks: int) -> bool:
        """One quantum: up to ``max_blocks`` vision blocks of the job under way (the next job is begun when one ends).
        True when every job of the plan has its visual embeddings."""
        while handle["next"] < len(handle["jobs"]):
            job = handle["jobs"][handle["next"]]
            if handle["encode"] is None:
                handle["encode"] = self.runners.call("begin_encode", job)
                if handle["encode"] is None:  # served from the visual-embedding cache
                    self._have_visual.add(job.seq_id)
                    handle["next"] += 1
                    continue
            handle["quanta"] += 1
            if not self.runners.call("advance_encode", handle["encode"], max_blocks):
                return False
            self._have_visual.add(job.seq_id)
            handle["encode"] = None
            handle["next"] += 1
            return handle["next"] == len(handle["jobs"])
        return True

    # ---- cooperative prefill: one prefill plan run a few decoder layers at a time (reference
    # ``engine/executor.py:35-95``: begin / advance / finish) ----------------------------------------
    def begin_prefill(self, plan: BatchPlan):
        """Page transfers, input preparation, vision tower and embedding of a prefill plan; the layers follow
        through ``advance_prefill``.  Returns the handle ``finish_prefill`` takes."""
        assert plan.phase is Phase.PREFILL
        t0 = time.perf_counter()
        if not plan.kv_transfers.empty:
            self.runners.call("apply_kv_transfers", plan.kv_transfers)
        with profile_region("engine.model_runner", metadata={"phase": "prefill_begin", "batch": plan.batch_size}):
            inputs = self.preparer.prepare(plan, self._have_visual)
            for job in inputs.vision_jobs:
                self._have_visual.add(job.seq_id)
            for sid in inputs.release_visual:
                self._have_visual.discard(sid)
            if self.attention_strategy:
                self._request_scores(plan, inputs)
            runner_handle = self.runners.call("begin_prefill", inputs)
        return {"plan": plan, "inputs": inputs, "runner": runner_handle, "ms": (time.perf_counter() - t0) * 1e3, "quanta": 0}

    def advance_prefill(self, handle, max_layers: int) -> bool:
        """Up to ``max_layers`` more decoder layers; True when every layer has run."""
        t0 = time.perf_counter()
        with profile_region("engine.model_runner", metadata={"phase": "prefill_quantum", "layers": max_layers}):
            done = bool(self.runners.call("advance_prefill", handle["runner"], int(max_layers)))
        handle["ms"] += (time.perf_counter() - t0) * 1e3
        handle["quanta"] += 1
        return done

    def finish_prefill(self, handle) -> ExecutionResult:
        """Whatever layers are left, the final norm and the first tokens of the plan's sequences."""
        t0 = time.perf_counter()
        plan, inputs = handle["plan"], handle["inputs"]
        with profile_region("engine.model_runner", metadata={"phase": "prefill_finish", "batch": plan.batch_size}):
            sampled = self.runners.call("finish_prefill", handle["runner"])
        tokens: list[int | None] = [None] * plan.batch_size
        for i, tok in zip(inputs.sample_seq, sampled):
            tokens[i] = int(tok)
        compactions = self._after_prefill(plan)
        return ExecutionResult(tuple(tokens), handle["ms"] + (time.perf_counter() - t0) * 1e3, compactions)

    def execute(self, plan: BatchPlan) -> ExecutionResult:
        t0 = time.perf_counter()
        if not plan.kv_transfers.empty:
            self.runners.call("apply_kv_transfers", plan.kv_transfers)
        if plan.is_idle:
            return ExecutionResult((), (time.perf_counter() - t0) * 1e3)
        with profile_region("engine.model_runner", metadata={"phase": plan.phase.value, "batch": plan.batch_size}):
            inputs = self.preparer.prepare(plan, self._have_visual)
            for job in inputs.vision_jobs:
                self._have_visual.add(job.seq_id)
            for sid in inputs.release_visual:
                self._have_visual.discard(sid)
            if self.attention_strategy and plan.phase is Phase.PREFILL:
                self._request_scores(plan, inputs)
            sampled = self.runners.call("execute", inputs)
        tokens: list[int | None] = [None] * plan.batch_size
        if plan.phase is Phase.PREFILL:
            for i, tok in zip(inputs.sample_seq, sampled):
                tokens[i] = int(tok)
        else:
            tokens = [int(t) for t in sampled]
        compactions = self._after_prefill(plan) if plan.phase is Phase.PREFILL else 0
        return ExecutionResult(tuple(tokens), (time.perf_counter() - t0) * 1e3, compactions)

    # ------------------------------------------------------------------------------
    def _whole_prompt(self, seq, sl) -> bool:
        return (seq.is_multimodal and sl.start == 0 and sl.end == len(seq) and seq.kv_layout is None and seq.num_cached_tokens == 0
                and 0 < seq.multimodal_prefix_boundary < len(seq))

    def _request_scores(self, plan: BatchPlan, inputs) -> None:
        """Ask the runner to score the sequences whose whole prompt is in this step."""
        row = 0
        for seq, sl in zip(plan.seqs, plan.slices):
            if self._whole_prompt(seq, sl):
                visual = tuple(i for span in seq.visual_spans for i in range(span.start, span.end))
                if visual:
                    inputs.score_rows.append((seq.seq_id, row, sl.length, visual))
            row += sl.length
        if inputs.score_rows:
            inputs.score_layers = list(self.score_layers)

    def _after_prefill(self, plan: BatchPlan) -> int:
        """Compaction and prefix publication for sequences whose chunk ended on the boundary."""
        plans = []
        owners = []
        scores = self.runners.call("take_visual_scores") if self.attention_strategy else None
        for seq, sl in zip(plan.seqs, plan.slices):
            boundary = seq.multimodal_prefix_boundary
            if scores and seq.seq_id in scores and scores[seq.seq_id] and self._whole_prompt(seq, sl):
                decision = compute_pruning_decision(seq.token_ids, seq.image_token_id, seq.video_token_id, self.pruning_scored,
                                                    end=boundary, scores=scores[seq.seq_id])
                self.attention_counters["scored"] += 1
                if decision is not None and decision.dropped:
                    seq.num_computed_tokens += sl.length
                    try:
                        cp = self.bm.build_compaction_plan(seq, retained_positions(boundary, decision), boundary)
                    finally:
                        seq.num_computed_tokens -= sl.length
                    if cp is not None:
                        plans.append(cp)
                        owners.append(seq)
                        seq.pruning_record = {"kept": len(decision.kept), "dropped": len(decision.dropped),
                                              "total": decision.total_visual_tokens, "strategy": "attention"}
                        self._record_decision(seq, decision, applied=True)
                continue
            if not seq.is_multimodal or boundary <= 0 or sl.end != boundary or sl.end >= len(seq):
                continue
            if self.compact and seq.kv_layout is None and seq.num_cached_tokens == 0:
                if self.attention_strategy:
                    self.attention_counters["uniform_fallback"] += 1
                decision = compute_pruning_decision(seq.token_ids, seq.image_token_id, seq.video_token_id, self.pruning,
                                                    end=boundary)
                if decision is not None and decision.dropped:
                    # the scheduler has not advanced num_computed_tokens yet
                    seq.num_computed_tokens += sl.length
                    try:
                        cp = self.bm.build_compaction_plan(seq, retained_positions(boundary, decision), boundary)
                    finally:
                        seq.num_computed_tokens -= sl.length
                    if cp is not None:
                        plans.append(cp)
                        owners.append(seq)
                        seq.pruning_record = {"kept": len(decision.kept), "dropped": len(decision.dropped),
                                              "total": decision.total_visual_tokens}
                        self._record_decision(seq, decision, applied=True)
        if self.shadow:
            # shadow mode: the selection a compacting mode would make, recorded when the prompt's prefix is complete;
            # the cache is left as it is (reference ``enable_visual_pruning_shadow``)
            for seq, sl in zip(plan.seqs, plan.slices):
                boundary = seq.multimodal_prefix_boundary
                if seq.is_multimodal and 0 < boundary and sl.start < boundary <= sl.end and seq.num_cached_tokens < boundary:
                    decision = compute_pruning_decision(seq.token_ids, seq.image_token_id, seq.video_token_id, self.pruning, end=boundary)
                    if decision is not None:
                        self._record_decision(seq, decision, applied=False)
        if plans:
            self.runners.call("compact_kv", plans)
            for seq, cp in zip(owners, plans):
                self.bm.commit_compaction(seq, cp)
                emit_kv_event("compact", seq_id=seq.seq_id, rows=len(cp.src_slots), released=len(cp.released_blocks))
        copies = []
        for seq, sl in zip(plan.seqs, plan.slices):
            boundary = seq.multimodal_prefix_boundary
            crossed = sl.end == boundary if self.compact else sl.start < boundary <= sl.end
            if seq.is_multimodal and boundary > 0 and crossed and seq.multimodal_prefix_cache_key:
                seq.num_computed_tokens += sl.length
                try:
                    copies.extend(self.bm.store_multimodal_prefix(seq))
                finally:
                    seq.num_computed_tokens -= sl.length
        if copies:
            self.runners.call("apply_kv_transfers", KVTransferPlan(copy_prefix=tuple(copies)))
        return len(plans)
