"""Pure host logic: config rules, request FSM, page pools, prefix caches, compaction,
scheduler policies, preemption.  No device, no checkpoint; tiny pages (4 tokens)."""

from types import SimpleNamespace

import pytest

from prism_infer_b200.config import Config, PrismConfig
from prism_infer_b200.engine.block_manager import BlockManager, chain_hash
from prism_infer_b200.engine.block_pool import CpuBlockPool, GpuBlockPool, OutOfBlocks
from prism_infer_b200.engine.compression import kv_bytes_per_token, traits
from prism_infer_b200.engine.contracts import BatchPlan, Phase
from prism_infer_b200.engine.kv_layout import CompactionPlan, KVLayout
from prism_infer_b200.engine.request import InvalidTransition, RequestLifecycle, RequestState
from prism_infer_b200.engine.scheduler import Scheduler
from prism_infer_b200.engine.scheduler_policy import FCFSPolicy, SLOAwarePolicy, VisionAwarePolicy
from prism_infer_b200.engine.sequence import Sequence
from prism_infer_b200.engine.visual_pruning import (PruningConfig, compute_pruning_decision, retained_positions,
                                                    target_keep_count, uniform_keep)
from prism_infer_b200.sampling_params import SamplingParams

IMG, VID, VS, VE, EOS = 901, 902, 903, 904, 905


def cfg(**kw):
    base = dict(max_num_seqs=8, max_num_batched_tokens=64, max_vision_patches_per_batch=4096, max_model_len=256, eos=EOS,
                num_kvcache_blocks=32, kvcache_block_size=4, num_cpu_blocks=0, enable_prefix_caching=True,
                compacts_visual_tokens=False, scheduler_policy="fcfs", max_queue_size=None, enable_chunked_prefill=True,
                max_chunk_size=16, max_consecutive_prefill_batches=1, heavy_prefill_vision_patch_threshold=64,
                min_decode_batches_between_heavy_prefills=3, max_light_prefill_bypasses_per_heavy=1)
    base.update(kw)
    return SimpleNamespace(**base)


def text_seq(i, n, max_tokens=4, base=10, **kw):
    return Sequence(i, list(range(base, base + n)), SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw),
                    image_token_id=IMG, video_token_id=VID)


def mm_seq(i, n_visual, question, key="media-A", max_tokens=4):
    ids = [VS] + [IMG] * n_visual + [VE] + list(question)
    s = Sequence(i, ids, SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True), image_token_id=IMG,
                 video_token_id=VID, image_grid_thw=[(1, 2, 2 * n_visual)], merge_size=2)
    s.multimodal_prefix_cache_key = key
    return s


# ------------------------------------------------------------------------------ config
def test_flat_config_adapter_rules():
    with pytest.raises(TypeError, match="unknown Prism config option"):
        PrismConfig.from_flat_options("random:tiny", {"no_such_knob": 1})
    c = PrismConfig.from_flat_options("random:tiny", {"kvcache_block_size": 64, "num_kvcache_blocks": 10,
                                                      "compression_mode": "scaled_fp8_kv"})
    assert c.cache.page_size == 64 and c.cache.num_gpu_blocks == 10 and c.execution.backend == "cuda_graph"
    assert c.quantization.kv_dtype == "fp8_e4m3" and c.quantization.kv_scaled
    assert PrismConfig.from_flat_options("random:tiny", {"enforce_eager": True}).execution.backend == "eager"
    with pytest.raises(ValueError, match="conflicts"):
        PrismConfig.from_flat_options("random:tiny", {"enforce_eager": True, "execution_backend": "cuda_graph"})
    with pytest.raises(ValueError, match="mutually exclusive"):
        PrismConfig.from_flat_options("random:tiny", {"decode_compile_region": "attention"})
    with pytest.raises(ValueError, match="logits_precision"):
        PrismConfig.from_flat_options("random:tiny", {"tensor_parallel_size": 2, "logits_precision": "fp32"})
    with pytest.raises(ValueError, match="eager-only"):
        PrismConfig.from_flat_options("random:tiny", {"compression_mode": "visual_prune"})
    with pytest.raises(ValueError):
        PrismConfig.from_flat_options("random:tiny", {"kvcache_block_size": 48})
    with pytest.raises(ValueError):
        PrismConfig.from_flat_options("/no/such/dir", {})
    with pytest.raises(ValueError, match="does not divide"):
        Config("random:tiny", tensor_parallel_size=3)


def test_start_up_validation_names_every_unmet_requirement():
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.runtime_capabilities import (CapabilityReport, validate_runtime_capabilities,
                                                       validate_tensor_parallel_environment)

    ok = CapabilityReport("2.11.0", True, "NVIDIA B200", (10, 0), True, True, True)
    assert validate_runtime_capabilities(True, execution_backend="cuda_graph", compression_mode="scaled_fp8_kv", report=ok) is ok
    bare = CapabilityReport("2.11.0", True, "NVIDIA B200", (10, 0), True, False, False)
    with pytest.raises(RuntimeError, match="CUDA graphs.*float8_e4m3fn"):
        validate_runtime_capabilities(True, execution_backend="cuda_graph", compression_mode="scaled_fp8_kv", report=bare)
    validate_runtime_capabilities(True, execution_backend="eager", compression_mode="off", report=bare)
    arch = Qwen3VLArch.qwen3_vl_8b()
    validate_tensor_parallel_environment(arch, 8, 8, world_size=8)
    with pytest.raises(RuntimeError, match="only 4 are available"):
        validate_tensor_parallel_environment(arch, 8, 4)
    with pytest.raises(RuntimeError, match="WORLD_SIZE=2"):
        validate_tensor_parallel_environment(arch, 4, 8, world_size=2)
    with pytest.raises(ValueError):
        validate_tensor_parallel_environment(arch, 3, 8)


def test_kv_page_accounting_matches_reference_numbers():
    c8 = Config("random:qwen3-vl-8b", compression_mode="scaled_fp8_kv")
    assert c8.kv_bytes_per_page() == 19_464_192  # 18 874 368 payload + 589 824 scales
    assert c8.kv_bytes_per_page() * 220 == 4_282_122_240
    assert kv_bytes_per_token(36, 8, 128, 2) / kv_bytes_per_token(36, 8, 128, 0) == 0.515625
    assert Config("random:qwen3-vl-8b", compression_mode="scaled_fp8_kv", tensor_parallel_size=8).kv_bytes_per_page() * 8 == 19_464_192
    assert traits("visual_compact_scaled_fp8").compacts and traits("visual_prune").logical_prune


# ------------------------------------------------------------------------- request FSM
def test_request_lifecycle_transitions():
    lc = RequestLifecycle(1)
    lc.transition(RequestState.PREFILLING)
    lc.transition(RequestState.DECODING)
    lc.transition(RequestState.SWAPPED, "preempt")
    lc.transition(RequestState.DECODING)
    lc.transition(RequestState.FINISHED, "eos")
    assert lc.finish_reason == "eos" and len(lc.history) == 5
    with pytest.raises(InvalidTransition):
        lc.transition(RequestState.DECODING)
    with pytest.raises(InvalidTransition):
        RequestLifecycle(2).transition(RequestState.DECODING)
    r = RequestLifecycle(3)
    r.transition(RequestState.REJECTED, "too long")
    assert r.state.terminal


# ------------------------------------------------------------------------------- pools
def test_gpu_pool_refcounts_and_hash_revival():
    pool = GpuBlockPool(3)
    a = pool.allocate()
    pool.publish(a, 123, (1, 2, 3, 4))
    pool.release(a)
    assert pool.num_free == 3 and pool.lookup(123, (1, 2, 3, 4)) == a  # freed but still findable
    pool.retain(a)  # revive
    assert pool.num_free == 2 and pool.blocks[a].ref_count == 1
    assert pool.lookup(123, (9, 9, 9, 9)) is None  # token check guards collisions
    b, c = pool.allocate(), pool.allocate()
    with pytest.raises(OutOfBlocks):
        pool.allocate()
    pool.release(b)
    with pytest.raises(RuntimeError):
        pool.release(b)
    assert {a, b, c} == {0, 1, 2}
    cpu = CpuBlockPool(2)
    with pytest.raises(OutOfBlocks):
        cpu.allocate_many(3)
    assert cpu.num_free == 2  # all-or-nothing


# ----------------------------------------------------------------------- block manager
def test_text_prefix_sharing_append_and_cow():
    bm = BlockManager(16, 4)
    s1, s2 = text_seq(1, 10), text_seq(2, 10)
    bm.allocate(s1)
    assert s1.num_cached_tokens == 0 and len(s1.block_table) == 3
    early = text_seq(9, 10)
    bm.allocate(early)  # s1's pages hold no KV yet: nothing to share
    assert early.num_cached_tokens == 0 and not set(early.block_table) & set(s1.block_table)
    bm.deallocate(early)
    s1.num_computed_tokens = 10
    assert bm.publish_computed_pages(s1) == 2 and not s1.unpublished_hashes
    bm.allocate(s2)
    assert s2.num_cached_tokens == 8 and s2.block_table[:2] == s1.block_table[:2] and s2.block_table[2] != s1.block_table[2]
    exact = text_seq(3, 8)
    bm.allocate(exact)  # all pages would hit, but the last token must be computed
    assert exact.num_cached_tokens == 4
    s1.append_token(5)
    s1.append_token(6)  # 12 tokens: KV row 11 still fits in page 2
    assert not bm.needs_new_page(s1)
    s1.append_token(7)  # 13 tokens: row 12 opens page 3
    assert bm.needs_new_page(s1) and bm.append(s1) == () and len(s1.block_table) == 4
    shared = s1.block_table[0]
    pair = bm.copy_on_write(s1, 0)
    assert pair[0] == shared and s1.block_table[0] == pair[1] and bm.gpu.blocks[shared].ref_count == 2
    for s in (s1, s2, exact):
        bm.deallocate(s)
    assert bm.gpu.num_free == 16


def test_swap_out_and_in_restore_hashes():
    bm = BlockManager(4, 4, num_cpu_blocks=4)
    s = text_seq(1, 8)
    bm.allocate(s)
    s.num_computed_tokens = 8
    bm.publish_computed_pages(s)
    hashes = [bm.gpu.blocks[b].hash for b in s.block_table]
    assert all(h is not None for h in hashes)
    out_pairs = bm.swap_out(s)
    assert len(out_pairs) == 2 and not s.block_table and len(s.cpu_block_table) == 2 and bm.gpu.num_free == 4
    filler = text_seq(2, 16)
    bm.allocate(filler)
    assert not bm.can_swap_in(s)
    bm.deallocate(filler)
    in_pairs = bm.swap_in(s)
    assert len(in_pairs) == 2 and bm.cpu.num_free == 4
    assert [bm.gpu.blocks[b].hash for b in s.block_table][0] in hashes + [None]


def test_multimodal_prefix_store_hit_tail_clone_and_eviction():
    bm = BlockManager(12, 4)
    a = mm_seq(1, 5, [50, 51, 52])  # prefix = VS + 5 IMG = 6 tokens -> 1 full page + 2 tail rows
    assert a.multimodal_prefix_boundary == 6 and bm.probe_multimodal_prefix(a) is None
    bm.allocate(a)
    assert a.num_cached_tokens == 0  # multimodal prompts never share by token hash
    a.num_computed_tokens = 6
    copies = bm.store_multimodal_prefix(a)
    assert len(copies) == 1 and copies[0][0] == a.block_table[1] and copies[0][2] == 2  # tail clone of 2 rows
    entry = next(iter(bm.entries.values()))
    assert entry.prefix_len == 6 and entry.tail_rows == 2 and entry.pages[0] == a.block_table[0]
    b = mm_seq(2, 5, [60, 61])
    assert bm.probe_multimodal_prefix(b) is entry
    plan = bm.allocate(b)
    assert b.num_cached_tokens == 6 and b.num_computed_tokens == 6 and b.block_table[0] == a.block_table[0]
    assert plan.copy_prefix == ((entry.pages[1], b.block_table[1], 2),)
    other = mm_seq(3, 5, [60, 61], key="media-B")
    assert bm.probe_multimodal_prefix(other) is None
    bm.deallocate(a)
    bm.deallocate(b)
    assert bm.gpu.num_free == 12 - 2  # the cache still holds its two pages
    big = text_seq(4, 44)  # needs 11 pages -> forces eviction of the entry
    bm.allocate(big)
    assert not bm.entries and bm.counters.evictions == 1
    stale = mm_seq(5, 5, [1])
    bm.deallocate(big)
    bm.allocate(stale, expected_hit=True)
    assert bm.counters.stale_probes == 1 and stale.num_cached_tokens == 0


def test_eviction_skips_entries_whose_pages_are_all_borrowed():
    """An entry whose pages are all still held by running sequences frees nothing when evicted: it
    stays in the cache, and the pool reports no reclaimable page for it."""
    bm = BlockManager(4, 4)
    a = mm_seq(1, 8, [5])  # vision_start + 8 placeholders: two full pages + a one-row tail; 11 tokens in all
    assert a.multimodal_prefix_boundary % 4 == 1 and len(a) <= 12
    bm.allocate(a)
    a.num_computed_tokens = len(a)
    bm.store_multimodal_prefix(a)  # takes the fourth page for the tail clone
    assert bm.gpu.num_free == 0 and bm._evictable_pages() == 1
    events = []
    from prism_infer_b200.observability import install_kv_trace_provider
    install_kv_trace_provider(lambda kind, fields: events.append(kind))
    try:
        assert bm._ensure_free(1) and not bm.entries and bm.counters.evictions == 1  # the tail clone was reclaimable
        bm.store_multimodal_prefix(a)
        entry = next(iter(bm.entries.values()))
        bm.gpu.retain(entry.pages[-1])  # pretend a sequence borrows the tail clone as well
        bm._evictable -= 1
        assert bm._evictable_pages() == 0
        assert not bm._ensure_free(1) and len(bm.entries) == 1 and bm.counters.evictions == 1  # nothing to gain: kept
    finally:
        install_kv_trace_provider(None)
    assert events.count("evict") == 1 and "prefix_store" in events


def test_compaction_plan_commit_and_layout():
    bm = BlockManager(16, 4)
    s = mm_seq(1, 12, [70, 71, 72])  # prefix 13 tokens, prompt 17 tokens -> 5 pages
    bm.allocate(s)
    s.num_computed_tokens = 13
    dec = compute_pruning_decision(s.token_ids, IMG, VID, PruningConfig(0.5, 2), end=13)
    keep = retained_positions(13, dec)
    assert len(dec.kept) == 6 and keep[0] == 0 and len(keep) == 7
    plan = bm.build_compaction_plan(s, keep, 13)
    assert isinstance(plan, CompactionPlan) and plan.layout.dropped == 6
    assert len(plan.kept_blocks) == 3 and len(plan.released_blocks) == 2  # 17 - 6 = 11 rows -> 3 pages
    assert plan.dst_slots[:4] == tuple(s.block_table[0] * 4 + i for i in range(4))
    free_before = bm.gpu.num_free
    table_before = list(s.block_table)
    bm.commit_compaction(s, plan)
    assert bm.gpu.num_free == free_before + 2 and s.block_table == table_before[:3]
    assert s.physical_len() == 11 and s.slot_of(13) == s.block_table[1] * 4 + 3  # logical 13 -> physical 7
    with pytest.raises(RuntimeError, match="stale"):
        bm.commit_compaction(s, plan)
    with pytest.raises(ValueError):
        KVLayout(5, (0, 2, 2))
    with pytest.raises(ValueError):
        KVLayout(5, (0, 7))
    copies = bm.store_multimodal_prefix(s)
    entry = next(iter(bm.entries.values()))
    assert entry.layout is s.kv_layout and entry.physical_len == 7 and copies[0][2] == 3
    hit = mm_seq(2, 12, [80])
    bm.allocate(hit)
    assert hit.kv_layout is s.kv_layout and hit.physical_len() == len(hit) - 6


# ------------------------------------------------------------------------- pruning math
def test_pruning_keep_counts_and_uniform_selection():
    assert target_keep_count(1568, 768, 0.6) == 941 and target_keep_count(1000, 768, 0.6) == 768
    assert target_keep_count(500, 768, 0.6) == 500 and target_keep_count(0, 32, 0.6) == 0
    idx = list(range(100, 120))
    kept = uniform_keep(idx, 5)
    assert kept[0] == 100 and kept[-1] == 119 and len(kept) == 5 and list(kept) == sorted(kept)
    assert uniform_keep(idx, 1) == (110,) and uniform_keep(idx, 50) == tuple(idx)
    video_only = [VS] + [VID] * 40 + [VE]
    assert compute_pruning_decision(video_only, IMG, VID, PruningConfig(0.5, 4)).dropped == ()  # video floor unset
    assert len(compute_pruning_decision(video_only, IMG, VID, PruningConfig(0.5, 4, 10)).kept) == 20
    scores = {i: float(i % 7) for i in range(1, 41)}
    d = compute_pruning_decision(video_only, IMG, VID, PruningConfig(0.25, 4, 4, "score"), scores=scores)
    assert len(d.kept) == 10 and all(scores[i] >= 5 for i in d.kept)


# --------------------------------------------------------------------------- scheduler
def run_step(sched, tokens=None):
    plan = sched.schedule()
    if plan.is_idle:
        return plan, []
    toks = tokens if tokens is not None else [7] * plan.batch_size
    return plan, sched.postprocess(plan, toks)


def test_scheduler_admission_chunking_and_finish():
    sched = Scheduler(cfg())
    too_long = text_seq(1, 300)
    assert not sched.add(too_long) and too_long.state is RequestState.REJECTED and sched.counters["rejected"] == 1
    wide = mm_seq(2, 40, [1])  # one visual span wider than the chunk limit
    assert not sched.add(wide)
    s = text_seq(3, 40, max_tokens=2)
    assert sched.add(s)
    plan, outs = run_step(sched)
    assert plan.phase is Phase.PREFILL and plan.slices[0].length == 16 and outs[0].new_token is None
    run_step(sched)
    plan, outs = run_step(sched)
    assert plan.slices[0].start == 32 and plan.slices[0].length == 8 and outs[0].new_token == 7
    assert s.state is RequestState.DECODING
    plan, outs = run_step(sched)
    assert plan.phase is Phase.DECODE and outs[0].finished and outs[0].finish_reason == "length"
    assert sched.is_finished() and sched.block_manager.gpu.num_free == 32
    e = text_seq(4, 5, max_tokens=9)
    sched.add(e)
    run_step(sched)
    _, outs = run_step(sched, [EOS])
    assert outs[0].finish_reason == "eos"


def test_text_prefix_pages_are_shared_only_once_computed():
    """Two identical long prompts under chunked prefill, and a cancel in mid-prefill followed by
    a resubmission: a page's content hash becomes visible only after the chunk that fills it ran."""
    sched = Scheduler(cfg(max_num_batched_tokens=32, max_chunk_size=8))
    a, b = text_seq(1, 30, max_tokens=1), text_seq(2, 33, max_tokens=1)  # same first 30 tokens
    sched.add(a)
    sched.add(b)
    plan, _ = run_step(sched)
    assert plan.phase is Phase.PREFILL and [s.seq_id for s in plan.seqs] == [1, 2]
    # b was admitted while a's pages were still empty: no cached tokens, no shared pages
    assert b.num_cached_tokens == 0 and not set(a.block_table) & set(b.block_table)
    assert all(sl.start + sl.length <= s.num_computed_tokens for s, sl in zip(plan.seqs, plan.slices))
    bm = sched.block_manager
    published = {blk.hash for blk in bm.gpu.blocks if blk.hash is not None}
    assert len(published) == 2  # the two pages the first 8-token chunk filled, once
    while not sched.is_finished():
        run_step(sched)
    # a third identical prompt arrives after everything was computed: full-page hits
    c = text_seq(3, 30, max_tokens=1)
    sched.add(c)
    run_step(sched)
    assert c.num_cached_tokens == 28
    while not sched.is_finished():
        run_step(sched)
    assert bm.gpu.num_free == 32

    # cancel after the first chunk: only the computed pages keep a hash
    sched = Scheduler(cfg(max_num_batched_tokens=8, max_chunk_size=8))
    bm = sched.block_manager
    d = text_seq(4, 30, max_tokens=1, base=500)
    sched.add(d)
    run_step(sched)
    assert d.num_computed_tokens == 8
    pages = list(d.block_table)
    sched.cancel(4)
    assert [bm.gpu.blocks[p].hash is not None for p in pages] == [True, True] + [False] * 6
    e = text_seq(5, 30, max_tokens=1, base=500)
    sched.add(e)
    plan, _ = run_step(sched)
    assert e.num_cached_tokens == 8 and plan.slices[0].start == 8  # revives the two computed pages only
    while not sched.is_finished():
        run_step(sched)
    assert bm.gpu.num_free == 32


def test_chunks_never_split_visual_spans_and_stop_at_prefix():
    pol = FCFSPolicy(cfg(max_chunk_size=16))
    s = mm_seq(1, 10, list(range(20)))  # VS, 10 IMG, VE, 20 text; boundary = 11
    assert pol.prefill_token_count(s, 64, stop_at_prefix=True) == 11
    assert pol.prefill_token_count(s, 64, stop_at_prefix=False) == 16
    assert pol.prefill_token_count(s, 5, stop_at_prefix=False) == 1  # only VS fits before the span
    s.num_computed_tokens = 1
    assert pol.prefill_token_count(s, 5, stop_at_prefix=False) == 0  # the span does not fit the budget
    assert pol.prefill_token_count(s, 12, stop_at_prefix=True) == 10
    two = Sequence(2, [VS] + [IMG] * 6 + [VE] + [5, 6] + [VS] + [IMG] * 6 + [VE] + [9], SamplingParams(),
                   image_token_id=IMG, video_token_id=VID)
    assert pol.prefill_token_count(two, 64, stop_at_prefix=False) == 11  # would cut the second span at 16


def test_lifo_preemption_recompute_and_swap():
    sched = Scheduler(cfg(num_kvcache_blocks=4, max_chunk_size=64))
    a, b = text_seq(1, 7, max_tokens=20, ignore_eos=True), text_seq(2, 7, max_tokens=20, base=500, ignore_eos=True)
    sched.add(a)
    sched.add(b)
    run_step(sched)  # both prefill: 2 pages each, pool full
    assert sched.block_manager.gpu.num_free == 0
    plan, _ = run_step(sched)  # a and b at 8 tokens: row 7 fits
    assert plan.phase is Phase.DECODE and plan.batch_size == 2
    plan, _ = run_step(sched)  # 9 tokens each: both need a page -> b (last in) is preempted by recompute
    assert sched.counters["preempt_recompute"] == 1 and b.state is RequestState.WAITING and not b.block_table
    assert plan.seqs == (a,) and sched.waiting[0] is b and b.num_computed_tokens == 0
    sw = Scheduler(cfg(num_kvcache_blocks=4, num_cpu_blocks=8, max_chunk_size=64))
    a, b = text_seq(1, 7, max_tokens=20, ignore_eos=True), text_seq(2, 7, max_tokens=20, base=500, ignore_eos=True)
    sw.add(a)
    sw.add(b)
    run_step(sw)
    run_step(sw)
    plan, _ = run_step(sw)
    assert sw.counters["preempt_swap"] == 1 and b.state is RequestState.SWAPPED and len(plan.kv_transfers.swap_out) == 2
    assert sw.cancel(a.seq_id) and a.state is RequestState.CANCELLED
    plan, _ = run_step(sw)
    assert b.state is RequestState.DECODING and len(plan.kv_transfers.swap_in) == 2 and sw.counters["swap_in"] == 1


def test_cancel_in_every_queue_frees_pages():
    sched = Scheduler(cfg())
    w, r = text_seq(1, 6), text_seq(2, 6, max_tokens=50, ignore_eos=True)
    sched.add(r)
    run_step(sched)
    sched.add(w)
    assert sched.cancel(w.seq_id) and sched.cancel(r.seq_id) and not sched.cancel(99)
    assert sched.block_manager.gpu.num_free == 32 and sched.is_finished() and sched.counters["cancelled"] == 2


def test_vision_aware_and_slo_policies():
    c = cfg(scheduler_policy="vision_aware", max_chunk_size=64, max_num_batched_tokens=64)
    pol = VisionAwarePolicy(c)
    sched = Scheduler(c, policy=pol)
    dec = text_seq(1, 4, max_tokens=100, ignore_eos=True)
    sched.add(dec)
    run_step(sched)
    heavy = mm_seq(2, 20, [1, 2])  # 80 patches >= threshold 64
    light = text_seq(3, 4)
    pol.decode_batches_since_heavy = 0
    sched.add(heavy)
    sched.add(light)
    plan, _ = run_step(sched)
    assert plan.phase is Phase.DECODE  # prefill / decode alternation comes first
    plan, _ = run_step(sched)
    assert plan.phase is Phase.PREFILL and plan.seqs == (light,)  # light overtakes the blocked heavy head
    phases = []
    for _ in range(6):
        plan, _ = run_step(sched)
        phases.append(plan.phase)
    assert Phase.DECODE in phases[:3] and any(p is Phase.PREFILL for p in phases)  # heavy admitted after enough decodes
    slo = SLOAwarePolicy(cfg(scheduler_policy="slo_aware"))
    x, y, z = text_seq(1, 4), text_seq(2, 4), mm_seq(3, 20, [1])
    x.deadline_ns, y.deadline_ns, z.deadline_ns = 900_000_000, 300_000_000, 800_000_000
    q = [x, y, z]
    slo.order_waiting(q, 0)
    assert q == [z, y, x] and slo.cost_tier(z) == 2 and slo.cost_tier(x) == 0  # heavy vision reserves 700 ms


def test_batch_plan_contract():
    with pytest.raises(ValueError):
        BatchPlan(Phase.PREFILL, (text_seq(1, 3),), ())
    assert BatchPlan(Phase.IDLE).is_idle and chain_hash([1, 2], None) != chain_hash([1, 2], 5)


def test_engine_metrics_ledger_is_bounded_and_times_tokens():
    """Per-request TTFT / TPOT from an injected clock, and the ledger bound of a long-running
    server: the oldest request and batch records are dropped, the newest kept."""
    from prism_infer_b200.engine.contracts import BatchPlan, Phase
    from prism_infer_b200.engine.metrics import EngineMetrics
    from prism_infer_b200.engine.sequence import Sequence
    from prism_infer_b200.sampling_params import SamplingParams

    now = [0]
    m = EngineMetrics(clock_ns=lambda: now[0], max_records=3)
    seqs = [Sequence(i, [1, 2, 3], SamplingParams(max_tokens=4)) for i in range(5)]
    for i, s in enumerate(seqs):
        now[0] = i * 1_000_000
        m.on_request_submitted(s)
    assert list(m.requests) == [2, 3, 4]
    s = seqs[4]
    now[0] = 10_000_000
    m.on_request_scheduled(s)
    now[0] = 14_000_000
    m.on_tokens(s)                                   # first token 10 ms after arrival (arrival at 4 ms)
    for k in range(3):
        now[0] += 2_000_000
        m.on_tokens(s)
    m.on_request_finished(s)
    rec = [r for r in m.snapshot()["requests"] if r["request_id"] == 4][0]
    assert rec["ttft_ms"] == 10.0 and rec["tpot_ms"] == 2.0 and rec["output_tokens"] == 4 and rec["queue_ms"] == 6.0
    m.on_tokens(seqs[0])                             # a dropped request: ignored
    for k in range(7):
        m.on_batch_completed(BatchPlan(Phase.DECODE, (s,), (), num_tokens=1), float(k))
    batches = m.snapshot()["batches"]
    assert [b["duration_ms"] for b in batches] == [4.0, 5.0, 6.0]
    m.reset()
    assert m.snapshot() == {"requests": [], "batches": []}


def _check_page_invariants(sched):
    """Every GPU page's reference count equals the number of owners that name it (block tables of
    live sequences + multimodal prefix entries); free + used = total; no page is both free and
    referenced; CPU pages are owned exactly by the swapped sequences."""
    bm = sched.block_manager
    owners: dict[int, int] = {}
    live = list(sched.running) + list(sched.waiting) + list(sched.swapped)
    for s in live:
        for p in s.block_table:
            owners[p] = owners.get(p, 0) + 1
    for e in bm.entries.values():
        for p in e.pages:
            owners[p] = owners.get(p, 0) + 1
    free = set(bm.gpu.free)
    assert len(free) == len(bm.gpu.free), "a page is on the free list twice"
    for blk in bm.gpu.blocks:
        want = owners.get(blk.block_id, 0)
        if blk.block_id in free:
            assert want == 0, f"page {blk.block_id} is free but referenced {want}x"
        else:
            assert blk.ref_count == want, f"page {blk.block_id}: ref_count {blk.ref_count}, owners {want}"
    assert bm.gpu.num_free + len(owners) == bm.gpu.num_blocks
    cpu_owned = sum(len(getattr(s, "cpu_block_table", []) or []) for s in sched.swapped)
    assert bm.cpu.num_blocks - bm.cpu.num_free == cpu_owned
    for s in sched.running:
        assert s.state in (RequestState.PREFILLING, RequestState.DECODING)
    for s in sched.swapped:
        assert s.state is RequestState.SWAPPED and not s.block_table
    # the running count of reclaimable prefix pages equals a full recount
    assert bm._evictable_pages() == sum(1 for e in bm.entries.values() for p in e.pages if bm.gpu.blocks[p].ref_count == 1)
    assert bm._entry_pages == {p for e in bm.entries.values() for p in e.pages}


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("cpu_blocks", [0, 12])
def test_random_traffic_keeps_page_accounting_exact(seed, cpu_blocks):
    """Random arrivals (text with shared prefixes, multimodal with repeated media), random
    cancellations and random tokens (EOS included) on a pool small enough to force preemption,
    swapping, prefix eviction and copy-on-write: the page accounting holds after every step
    and every page is free at the end."""
    import random

    rng = random.Random(seed)
    sched = Scheduler(cfg(num_kvcache_blocks=14, num_cpu_blocks=cpu_blocks, max_num_seqs=5, max_num_batched_tokens=48,
                          compacts_visual_tokens=False))
    next_id = 0
    submitted = 0
    for step in range(400):
        if submitted < 60 and rng.random() < 0.45:
            next_id += 1
            submitted += 1
            if rng.random() < 0.5:
                seq = text_seq(next_id, rng.randint(3, 22), max_tokens=rng.randint(1, 12), base=rng.choice([10, 10, 50]))
            else:
                seq = mm_seq(next_id, rng.choice([4, 8]), [rng.randint(1, 800) for _ in range(rng.randint(1, 5))],
                             key=rng.choice(["media-A", "media-B", "media-C"]), max_tokens=rng.randint(1, 10))
            sched.add(seq)
        if rng.random() < 0.08:
            live = list(sched.running) + list(sched.waiting) + list(sched.swapped)
            if live:
                sched.cancel(rng.choice(live).seq_id)
        plan = sched.schedule()
        if not plan.is_idle:
            toks = [EOS if rng.random() < 0.05 else rng.randint(1, 800) for _ in range(plan.batch_size)]
            if plan.phase is Phase.PREFILL:  # what the executor does after a prefill: publish crossed prefixes
                outs = None
                for seq, sl in zip(plan.seqs, plan.slices):
                    b = seq.multimodal_prefix_boundary if seq.is_multimodal else 0
                    if b > 0 and sl.start < b <= sl.end and seq.multimodal_prefix_cache_key:
                        seq.num_computed_tokens += sl.length
                        try:
                            sched.block_manager.store_multimodal_prefix(seq)
                        finally:
                            seq.num_computed_tokens -= sl.length
            sched.postprocess(plan, toks)
        _check_page_invariants(sched)
        if submitted >= 60 and sched.is_finished():
            break
    for _ in range(300):  # drain
        if sched.is_finished():
            break
        plan = sched.schedule()
        if not plan.is_idle:
            sched.postprocess(plan, [EOS] * plan.batch_size)
        _check_page_invariants(sched)
    assert sched.is_finished()
    bm = sched.block_manager
    held = sum(len(e.pages) for e in bm.entries.values())
    assert bm.gpu.num_free + held == bm.gpu.num_blocks and bm.cpu.num_free == bm.cpu.num_blocks
    TRAFFIC_COUNTERS.append((dict(sched.counters), dict(bm.counters.snapshot())))


TRAFFIC_COUNTERS: list = []


def test_random_traffic_reached_the_interesting_paths():
    """The runs above, taken together, preempted by swap and by recompute, swapped back in,
    hit and evicted multimodal prefixes, and finished and cancelled requests."""
    if len(TRAFFIC_COUNTERS) < 12:
        pytest.skip("runs only after the whole random-traffic matrix")
    total: dict[str, int] = {}
    for sched_c, prefix_c in TRAFFIC_COUNTERS:
        for k, v in {**sched_c, **prefix_c}.items():
            if isinstance(v, int):
                total[k] = total.get(k, 0) + v
    for key in ("preempt_swap", "preempt_recompute", "swap_in", "finished", "cancelled", "hits", "stores", "evictions"):
        assert total.get(key, 0) > 0, (key, total)


def test_options_document_lists_every_flat_option():
    """``docs/OPTIONS.md`` is the generated table of ``LLM`` keywords: regenerate it when the
    configuration changes."""
    import os

    from prism_infer_b200.config import FLAT_OPTION_NAMES
    from prism_infer_b200.utils import describe_options

    rows = describe_options.option_rows()
    assert {r[0] for r in rows} == set(FLAT_OPTION_NAMES)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "docs", "OPTIONS.md")) as fh:
        assert fh.read() == describe_options.markdown(), "run: python -m prism_infer_b200.utils.describe_options > docs/OPTIONS.md"
    # options marked "no effect" exist, and nothing outside the configuration module reads their fields
    import re
    import subprocess

    field_of = {r[0]: r[2] for r in rows}
    assert set(describe_options.COMPATIBILITY_ONLY) <= set(field_of)
    for public in describe_options.COMPATIBILITY_ONLY:
        hits = subprocess.run(["grep", "-rlE", "--include=*.py", rf"\.{field_of[public]}\b", os.path.join(root, "prism_infer_b200")],
                              capture_output=True, text=True).stdout.split()  # attribute reads: config.<field>
        readers = [h for h in hits if not re.search(r"prism_infer_b200/(config|utils/describe_options)\.py$", h)]
        assert not readers, (public, readers)


def test_environment_check_reports_checkpoint_and_plan_problems(tmp_path, capsys):
    """The environment tool passes on a sound checkpoint directory, names every defect of a broken one, refuses a
    tensor-parallel size the model cannot be split into, and its exit status follows the errors (warnings do not)."""
    import json

    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.utils import check_environment as ce

    arch = Qwen3VLArch.tiny()
    good = tmp_path / "good"
    good.mkdir()
    (good / "config.json").write_text(json.dumps(arch.to_hf_config()))
    (good / "model.safetensors").write_bytes(b"\0" * 2048)
    rc = ce.main(["--allow-cpu", "--model", str(good), "--json"])
    rep = json.loads(capsys.readouterr().out)
    assert rc == 0 and rep["status"] == "pass" and rep["model"]["weight_files"] == 1 and rep["model"]["text"]["kv_heads"] == 2
    assert len(rep["model"]["config_sha256"]) == 64 and rep["kernel_library"]["path"].endswith("libprism_b200.so")
    assert any("tokenizer_config.json" in w for w in rep["warnings"])  # recommended, not required
    assert rep["planned_run"] == {"execution_backend": "cuda_graph", "compression_mode": "scaled_fp8_kv", "tensor_parallel_size": 1,
                                  "require_cuda": False}
    # two KV heads cannot be split over four ranks
    rc = ce.main(["--allow-cpu", "--model", str(good), "--tensor-parallel-size", "4", "--json"])
    rep = json.loads(capsys.readouterr().out)
    assert rc == 1 and any("configuration rejected" in e for e in rep["errors"])
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text(json.dumps({"model_type": "llama", "architectures": ["LlamaForCausalLM"]}))
    rc = ce.main(["--allow-cpu", "--model", str(bad), "--json"])
    rep = json.loads(capsys.readouterr().out)
    assert rc == 1 and any("no *.safetensors" in e for e in rep["errors"]) and any("does not describe a Qwen3-VL" in e for e in rep["errors"])
    assert ce.main(["--allow-cpu", "--model", str(tmp_path / "nowhere"), "--json"]) == 1
    capsys.readouterr()
    assert ce.main(["--allow-cpu", "--model", "random:nope", "--json"]) == 1
    capsys.readouterr()
    # without --allow-cpu a machine without a CUDA device fails; --min-free-gib needs a device to look at
    import torch

    if not torch.cuda.is_available():
        assert ce.main(["--model", "random:tiny", "--json"]) == 1
        rep = json.loads(capsys.readouterr().out)
        assert any("no CUDA device" in e for e in rep["errors"])
        assert ce.main(["--allow-cpu", "--min-free-gib", "1", "--json"]) == 1
        capsys.readouterr()
    assert ce.main(["--allow-cpu", "--model", "random:tiny"]) == 0
    assert "result: PASS" in capsys.readouterr().out


def test_checkpoint_processor_files_set_pixel_budgets_and_video_sampling(tmp_path):
    import json

    from prism_infer_b200.engine.vl_inputs import PatchProcessor, checkpoint_pixel_budgets
    from prism_infer_b200.models.architecture import Qwen3VLArch

    assert checkpoint_pixel_budgets(str(tmp_path)) == {}
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"min_pixels": 3136, "max_pixels": 1003520}))        # the older flat keys
    (tmp_path / "video_preprocessor_config.json").write_text(json.dumps({"size": {"shortest_edge": 4096, "longest_edge": 25165824},
                                                                         "fps": 2, "min_frames": 4, "max_frames": 768, "do_sample_frames": True}))
    got = checkpoint_pixel_budgets(str(tmp_path))
    assert got == {"min_pixels": 3136, "max_pixels": 1003520, "video_min_pixels": 4096, "video_max_pixels": 25165824, "video_fps": 2,
                   "video_min_frames": 4, "video_max_frames": 768}
    p = PatchProcessor(Qwen3VLArch.tiny(), **got)
    assert (p.min_pixels, p.max_pixels, p.video_fps, p.video_min_frames, p.video_max_frames) == (3136, 1003520, 2.0, 4, 768)
    (tmp_path / "preprocessor_config.json").write_text(json.dumps({"size": {"shortest_edge": 65536, "longest_edge": "many"}}))
    assert "max_pixels" not in checkpoint_pixel_budgets(str(tmp_path))  # a value that is not a number is ignored, not guessed


def test_shipped_configurations_and_a_configuration_written_for_the_reference_load():
    """Every file under ``configs/`` is a valid ``--engine-config``; and the option set of the reference's two-GPU graph
    configuration (``configs/tp2_graph.json`` there: its compile-and-graph backend and the switches of its fused
    kernels) loads unchanged, selects the graph backend here and changes nothing else."""
    import glob
    import os

    from prism_infer_b200.config import PrismConfig
    from prism_infer_b200.serving.cli import load_engine_options

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "configs", "*.json")))
    assert {os.path.basename(f) for f in files} >= {"tp2_graph.json", "tp8_graph.json"}
    for f in files:
        cfg = PrismConfig.from_flat_options("random:tiny", load_engine_options(f))
        assert cfg.execution.uses_graphs, f
    theirs = {"execution_backend": "compile_graph", "decode_compile_region": "attention", "decode_compile_mode": "default",
              "tensor_parallel_size": 2, "max_model_len": 1280, "max_num_batched_tokens": 2048, "max_num_seqs": 8,
              "gpu_memory_utilization": 0.9, "num_kvcache_blocks": 64, "enable_prefix_caching": True, "logits_precision": "model",
              "mlp_projection_mode": "packed", "paged_decode_block_n": 256, "enable_fused_qk_rmsnorm": True,
              "enable_fused_qk_mrope": True, "enable_fused_add_rmsnorm": True, "enable_packed_kv_projection": True}
    cfg = PrismConfig.from_flat_options("random:tiny", theirs)
    ours = PrismConfig.from_flat_options("random:tiny", load_engine_options(os.path.join(root, "configs", "tp2_graph.json")))
    assert cfg.execution.uses_graphs and cfg.scheduler == ours.scheduler and cfg.cache == ours.cache
    assert cfg.model.tensor_parallel_size == ours.model.tensor_parallel_size == 2
