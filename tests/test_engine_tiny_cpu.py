"""End-to-end slice on CPU: the tiny random-init Qwen3-VL through the public ``LLM`` API
against the plain-PyTorch oracle (one 224x224 image -> 196 patches -> 49 visual tokens,
24 random text ids, 16 greedy tokens)."""

import numpy as np
import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs, prepare_video_inputs
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.reference_model import ReferenceQwen3VL
from prism_infer_b200.models.weights import random_weights
from prism_infer_b200.utils.tokenizer import load_tokenizer


@pytest.fixture(scope="module")
def tiny():
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    return arch, weights, ReferenceQwen3VL(arch, weights)


def _image(seed=0, size=224):
    return np.random.default_rng(seed).integers(0, 256, (size, size, 3), dtype=np.uint8)


def _llm(weights, **kw):
    opts = dict(max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64, enforce_eager=True,
                max_num_batched_tokens=512, max_chunk_size=512)
    opts.update(kw)
    return LLM("random:tiny", weights=weights, device="cpu", **opts)


def test_image_prompt_matches_oracle(tiny):
    arch, weights, oracle = tiny
    g = torch.Generator().manual_seed(0)
    text = torch.randint(0, 1000, (24,), generator=g).tolist()
    inputs = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), text, [_image()])
    assert inputs.pixel_values.shape == (196, 1536) and sum(t == arch.image_token_id for t in inputs.input_ids) == 49
    want = oracle.generate_greedy(inputs.input_ids, 16, pixel_values=inputs.pixel_values,
                                  image_grid_thw=inputs.image_grid_thw)
    llm = _llm(weights)
    got = llm.generate_prepared_image_inputs(inputs, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    assert got["token_ids"] == want
    assert set(got) == {"text", "raw_text", "token_ids"}
    llm.exit()


@pytest.mark.parametrize("mode", ["off", "scaled_fp8_kv"])
def test_chunked_prefill_and_batching(tiny, mode):
    arch, weights, oracle = tiny
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (5, 40, 17)]
    llm = _llm(weights, max_chunk_size=16, compression_mode=mode)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    if mode == "off":
        for p, o in zip(prompts, outs):
            assert o["token_ids"] == oracle.generate_greedy(p, 8)
    else:
        assert all(len(o["token_ids"]) == 8 for o in outs)
    llm.exit()


def test_video_prompt_matches_oracle(tiny):
    arch, weights, oracle = tiny
    frames = [_image(s, 64) for s in range(4)]
    inputs = prepare_video_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [7, 8, 9, 10], frames)
    want = oracle.generate_greedy(inputs.input_ids, 6, pixel_values=inputs.pixel_values, video_grid_thw=inputs.video_grid_thw)
    llm = _llm(weights)
    got = llm.generate_prepared_video_inputs(inputs, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    assert got["token_ids"] == want
    llm.exit()


def test_prefix_cache_hit_reuses_visual_prefix(tiny):
    arch, weights, oracle = tiny
    img = _image(3)
    llm = _llm(weights)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    tok = load_tokenizer("random:tiny", arch)
    a = prepare_image_inputs(PatchProcessor(arch), tok, [11, 12, 13], [img])
    b = prepare_image_inputs(PatchProcessor(arch), tok, [21, 22, 23, 24], [img])
    first = llm.generate_prepared_image_inputs(a, sp)
    second = llm.generate_prepared_image_inputs(b, sp)
    meta = llm.multimodal_prefix_cache_metadata()
    assert meta["stores"] == 1 and meta["hits"] == 1 and meta["tokens_reused"] == 50
    assert first["token_ids"] == oracle.generate_greedy(a.input_ids, 4, pixel_values=a.pixel_values, image_grid_thw=a.image_grid_thw)
    assert second["token_ids"] == oracle.generate_greedy(b.input_ids, 4, pixel_values=b.pixel_values, image_grid_thw=b.image_grid_thw)
    reqs = llm.metrics_snapshot()["engine"]["requests"]
    assert reqs[1]["cached_tokens"] == 50
    llm.exit()


def test_cooperative_prefill_keeps_the_transfers_of_requests_admitted_after_the_quantum(tiny):
    """A decoding sequence, a cold image request (vision quantum first), then a prefix-hit request
    that arrives between the quantum and the re-planned prefill: its tail-page copy must run."""
    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    proc = PatchProcessor(arch)
    llm = _llm(weights, enable_cooperative_prefill=True)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    known, fresh = _image(5), _image(6)
    llm.generate_prepared_image_inputs(prepare_image_inputs(proc, tok, [11, 12, 13], [known]), sp)  # stores the prefix
    text = [3, 4, 5, 6, 7]
    t_id = llm.add_request(text, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    cold = prepare_image_inputs(proc, tok, [41, 42], [fresh])
    c_id = llm.add_prepared_image_request(cold, sp)
    for _ in range(4):  # the policy may run a decode batch first
        if llm.step_result().phase.value == "idle":
            break
    assert llm.cooperative_counters["vision_quanta"] == 1 and llm.request_state(c_id).value == "prefilling"
    hit = prepare_image_inputs(proc, tok, [21, 22, 23, 24], [known])
    h_id = llm.add_prepared_image_request(hit, sp)
    done = {}
    while not llm.is_finished():
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
    assert llm.multimodal_prefix_cache_metadata()["tail_clones"] >= 1
    assert done[t_id] == oracle.generate_greedy(text, 12)
    assert done[c_id] == oracle.generate_greedy(cold.input_ids, 4, pixel_values=cold.pixel_values, image_grid_thw=cold.image_grid_thw)
    assert done[h_id] == oracle.generate_greedy(hit.input_ids, 4, pixel_values=hit.pixel_values, image_grid_thw=hit.image_grid_thw)
    llm.exit()


def test_cooperative_prefill_runs_the_layers_in_quanta_between_decode_steps(tiny):
    """With a sequence decoding, a new prompt's prefill runs one decoder layer per quantum and every quantum is
    followed by a decode step of the running sequence; tokens equal the oracle's (and thus the atomic prefill's)."""
    arch, weights, oracle = tiny
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1)
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    late = list(range(40, 71))
    b_id = llm.add_request(late, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    phases, done = [], {}
    while not llm.is_finished():
        res = llm.step_result()
        phases.append((res.phase.value, llm.request_state(b_id).value if llm.request_state(b_id) else "gone"))
        for o in res.outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
    c = llm.cooperative_counters
    # two layers, one per quantum: begin, decode, layer 0, decode, layer 1 + final norm + first token
    assert c["layer_quantum_prefills"] == 1 and c["layer_quanta"] == arch.text.num_layers == 2
    assert c["decode_steps_between_quanta"] == 2
    # while B was prefilling, decode steps of A went through
    assert ("decode", "prefilling") in phases
    assert [p for p, _ in phases].count("prefill") == 1
    assert done[a_id] == oracle.generate_greedy(first, 14)
    assert done[b_id] == oracle.generate_greedy(late, 5)
    llm.exit()


def test_cancelling_a_request_whose_prefill_is_pending_drains_the_prefill_first(tiny):
    """The pages of a sequence in a pending prefill stay allocated until the remaining layers have written them: a
    cancel finishes the prefill, the other sequence of the same plan still gets its first token, nothing leaks."""
    arch, weights, oracle = tiny
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1)
    free0 = llm.scheduler.block_manager.gpu.num_free
    a_id = llm.add_request([3, 4, 5, 6, 7], SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    keep, drop = list(range(40, 60)), list(range(80, 105))
    k_id = llm.add_request(keep, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    d_id = llm.add_request(drop, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    done = {}
    for _ in range(6):
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
        if llm._pending_prefill is not None:
            break
    assert llm._pending_prefill is not None and {s.seq_id for s in llm._pending_prefill["plan"].seqs} == {k_id, d_id}
    assert llm.cancel_request(d_id) and llm._pending_prefill is None
    while not llm.is_finished():
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
    assert done[k_id] == oracle.generate_greedy(keep, 4) and d_id not in done
    assert done[a_id] == oracle.generate_greedy([3, 4, 5, 6, 7], 10)
    assert llm.scheduler.block_manager.gpu.num_free == free0
    llm.exit()


def _slo_engine(weights, now, **kw):
    # 196 patches (one 224 x 224 image) count as a heavy visual input here: cost tier 2
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1, scheduler_policy="slo_aware",
               num_kvcache_blocks=96, heavy_prefill_vision_patch_threshold=100, **kw)
    llm.scheduler.clock_ns = lambda: now[0]
    return llm


def _drain(llm, done):
    while not llm.is_finished():
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)


def test_a_due_cheaper_request_interrupts_a_pending_prefill(tiny):
    """SLO-aware policy: while a long prompt (cost tier 1) is prefilling by layer quanta, a short prompt (tier 0)
    whose release time has come gets its whole prefill at once; the running sequence decodes next, then the long
    prompt's quanta go on.  Every request's tokens equal the oracle's."""
    arch, weights, oracle = tiny
    now = [1_000_000_000]
    llm = _slo_engine(weights, now)
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    g = torch.Generator().manual_seed(7)
    long = torch.randint(0, 1000, (300,), generator=g).tolist()
    b_id = llm.add_request(long, SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    done = {}
    for _ in range(4):
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
        if llm._pending_prefill is not None:
            break
    assert llm._pending_prefill is not None and llm.scheduler.policy.cost_tier(llm._sequences[b_id]) == 1
    short = [9, 8, 7, 6]
    c_id = llm.add_request(short, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    seq_c = llm._sequences[c_id]
    seq_c.deadline_ns = now[0] + 200_000_000  # release in 80 ms (tier 0 reserves 120 ms): not due yet
    quanta_before = llm.cooperative_counters["decode_steps_between_quanta"]
    res = llm.step_result()
    assert llm.cooperative_counters["slo_prefill_interruptions"] == 0 and res.phase.value == "decode"
    now[0] += 100_000_000  # past the release time
    res = llm.step_result()
    assert res.phase.value == "prefill" and llm.cooperative_counters["slo_prefill_interruptions"] == 1
    assert llm.request_state(c_id).value == "decoding" and llm.request_state(b_id).value == "prefilling"
    assert llm._pending_prefill is not None
    res = llm.step_result()  # the sequences that were running decode before anything else
    assert res.phase.value == "decode" and llm.cooperative_counters["decode_steps_between_quanta"] == quanta_before + 2
    _drain(llm, done)
    assert done[a_id] == oracle.generate_greedy(first, 12)
    assert done[b_id] == oracle.generate_greedy(long, 3)
    assert done[c_id] == oracle.generate_greedy(short, 4)
    assert llm.cooperative_counters["slo_prefill_interruptions"] == 1
    llm.exit()


def _heavy_image_request(arch, seed=8):
    return prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [31, 32, 33], [_image(seed)])


def test_a_pending_prefill_whose_own_release_time_passes_finishes_in_one_piece(tiny):
    arch, weights, oracle = tiny
    now = [5_000_000_000]
    llm = _slo_engine(weights, now)
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    late = _heavy_image_request(arch)
    b_id = llm.add_prepared_image_request(late, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert llm.scheduler.policy.cost_tier(llm._sequences[b_id]) == 2
    llm._sequences[b_id].deadline_ns = now[0] + 2_000_000_000
    done = {}
    for _ in range(6):  # vision quantum, then the language prefill is begun
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
        if llm._pending_prefill is not None:
            break
    c = llm.cooperative_counters
    assert llm._pending_prefill is not None and c["slo_deadline_atomic_prefills"] == 0 and c["slo_light_atomic_prefills"] == 0
    now[0] += 1_400_000_000  # 600 ms before the deadline: inside the 700 ms reserve of a heavy request
    res = llm.step_result()
    assert res.phase.value == "prefill" and llm._pending_prefill is None and c["slo_pending_deadline_finishes"] == 1
    assert c["layer_quanta"] == 0  # no layer had run as a quantum: all of them ran in the finishing step
    _drain(llm, done)
    assert done[a_id] == oracle.generate_greedy(first, 10)
    assert done[b_id] == oracle.generate_greedy(late.input_ids, 4, pixel_values=late.pixel_values, image_grid_thw=late.image_grid_thw)
    llm.exit()


def test_a_prefill_that_is_already_due_or_cheap_does_not_yield_to_decode_steps(tiny):
    """Under the SLO-aware policy a heavy request past its release time runs in one piece, and so does a prompt of a
    cheap tier that carries a deadline at all (quanta would only delay its first token)."""
    arch, weights, oracle = tiny
    now = [5_000_000_000]
    llm = _slo_engine(weights, now)
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    heavy = _heavy_image_request(arch)
    b_id = llm.add_prepared_image_request(heavy, SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    llm._sequences[b_id].deadline_ns = now[0] + 50_000_000
    done = {}
    while llm.request_state(b_id) is not None and llm.request_state(b_id).value in ("waiting", "prefilling"):
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
    c = llm.cooperative_counters
    assert c["slo_deadline_atomic_prefills"] == 1 and c["layer_quantum_prefills"] == 0
    light = list(range(40, 71))
    l_id = llm.add_request(light, SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    llm._sequences[l_id].deadline_ns = now[0] + 10_000_000_000  # far away: only the tier decides
    _drain(llm, done)
    assert c["slo_light_atomic_prefills"] == 1 and c["layer_quantum_prefills"] == 0
    assert done[a_id] == oracle.generate_greedy(first, 12) and done[l_id] == oracle.generate_greedy(light, 3)
    assert done[b_id] == oracle.generate_greedy(heavy.input_ids, 3, pixel_values=heavy.pixel_values, image_grid_thw=heavy.image_grid_thw)
    llm.exit()


def test_waiting_requests_are_coalesced_into_one_prefill_while_sequences_decode(tiny):
    """Adaptive cooperative prefill: one waiting request is held back (decode steps go on) until a third arrives or
    the oldest has waited long enough; three run as one atomic prefill; a lone request past the wait runs atomically
    while the engine is lightly loaded and in layer quanta once the decode batch has reached a quarter of the limit."""
    arch, weights, oracle = tiny
    now = [1_000_000_000]
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1, cooperative_prefill_coalesce_ms=250.0,
               max_num_seqs=8, num_kvcache_blocks=96)
    llm.scheduler.clock_ns = lambda: now[0]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)

    def add(prompt):
        rid = llm.add_request(prompt, sp)
        llm._sequences[rid].arrival_ns = now[0]
        return rid

    prompts = {}
    first = [3, 4, 5, 6, 7]
    prompts[add(first)] = first
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    c = llm.cooperative_counters
    for k in range(2):
        p = list(range(40 + 10 * k, 60 + 10 * k))
        prompts[add(p)] = p
    for _ in range(3):
        assert llm.step_result().phase.value == "decode"
    assert c["coalesce_deferred_decode_steps"] == 3 and len(llm.scheduler.waiting) == 2
    p = list(range(90, 120))
    prompts[add(p)] = p                      # the third waiting request: no more holding back
    res = llm.step_result()
    assert res.phase.value == "prefill" and res.num_tokens == 20 + 20 + 30 and c["coalesced_atomic_prefills"] == 1
    assert llm._pending_prefill is None and llm.scheduler.num_decoding == 4
    # a lone request: held for 250 ms, then (four sequences decode = a quarter of eight: the engine counts as loaded) in quanta
    p = list(range(200, 240))
    lone = add(p)
    prompts[lone] = p
    assert llm.step_result().phase.value == "decode" and c["coalesce_deferred_decode_steps"] == 4
    now[0] += 251_000_000
    llm.step_result()
    assert c["layer_quantum_prefills"] == 1 and c["underfilled_atomic_prefills"] == 0 and llm._pending_prefill is not None
    done = {}
    _drain(llm, done)
    for rid, prompt in prompts.items():
        assert done[rid] == oracle.generate_greedy(prompt, 30), rid
    llm.exit()


def test_a_lone_prefill_on_a_lightly_loaded_engine_runs_atomically_and_a_deadline_ends_the_wait(tiny):
    arch, weights, oracle = tiny
    now = [1_000_000_000]
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1, cooperative_prefill_coalesce_ms=250.0,
               max_num_seqs=8, num_kvcache_blocks=96, scheduler_policy="slo_aware")
    llm.scheduler.clock_ns = lambda: now[0]
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    c = llm.cooperative_counters
    late = list(range(40, 71))
    b_id = llm.add_request(late, SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    llm._sequences[b_id].arrival_ns = now[0]
    assert llm.step_result().phase.value == "decode" and c["coalesce_deferred_decode_steps"] == 1
    now[0] += 251_000_000
    assert llm.step_result().phase.value == "prefill"   # one decoder of eight: not loaded, so no quanta
    assert c["underfilled_atomic_prefills"] == 1 and c["layer_quantum_prefills"] == 0 and c["coalesce_deadline_releases"] == 0
    # a waiting request whose release time (deadline - 120 ms reserve) comes before the 250 ms are over
    third = list(range(80, 100))
    c_id = llm.add_request(third, SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    llm._sequences[c_id].arrival_ns = now[0]
    llm._sequences[c_id].deadline_ns = now[0] + 170_000_000
    assert llm.step_result().phase.value == "decode"
    now[0] += 60_000_000
    assert llm.step_result().phase.value == "prefill" and c["coalesce_deadline_releases"] == 1
    done = {}
    _drain(llm, done)
    assert done[a_id] == oracle.generate_greedy(first, 12) and done[b_id] == oracle.generate_greedy(late, 3)
    assert done[c_id] == oracle.generate_greedy(third, 3)
    llm.exit()


def test_cooperative_prefill_runs_the_vision_tower_in_block_quanta(tiny):
    """With a sequence decoding, the vision tower of a new image request runs one block per quantum with a decode step
    after every quantum, then the language prefill in layer quanta; tokens equal the oracle's.  A request cancelled
    while its tower is half run leaves nothing behind."""
    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1, cooperative_prefill_vision_block_quantum=1)
    free0 = llm.scheduler.block_manager.gpu.num_free
    first = [3, 4, 5, 6, 7]
    a_id = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    while llm.scheduler.num_decoding == 0:
        llm.step_result()
    img = prepare_image_inputs(PatchProcessor(arch), tok, [41, 42], [_image(9)])
    b_id = llm.add_prepared_image_request(img, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    phases, done = [], {}
    while llm.request_state(b_id) is not None and llm.request_state(b_id).value in ("waiting", "prefilling"):
        res = llm.step_result()
        phases.append(res.phase.value)
        for o in res.outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
    c = llm.cooperative_counters
    assert c["vision_block_quanta"] == arch.vision.depth == 2 and c["vision_quanta"] == 1 and c["layer_quantum_prefills"] == 1
    # quantum (idle), decode, quantum (idle), then the prefill is begun with a decode step, layer quanta follow
    assert phases[:4] == ["idle", "decode", "idle", "decode"] or phases[:5] == ["decode", "idle", "decode", "idle", "decode"], phases
    # a second image request is cancelled after its first block quantum
    img2 = prepare_image_inputs(PatchProcessor(arch), tok, [43, 44], [_image(10)])
    c_id = llm.add_prepared_image_request(img2, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    for _ in range(6):
        llm.step_result()
        if llm._pending_vision is not None:
            break
    assert llm._pending_vision is not None
    assert llm.cancel_request(c_id) and llm._pending_vision is None
    _drain(llm, done)
    assert c_id not in done
    assert done[a_id] == oracle.generate_greedy(first, 24)
    assert done[b_id] == oracle.generate_greedy(img.input_ids, 4, pixel_values=img.pixel_values, image_grid_thw=img.image_grid_thw)
    kept = llm.multimodal_prefix_cache_metadata()["resident_pages"]  # the first image's prefix stays cached
    assert kept > 0 and llm.scheduler.block_manager.gpu.num_free == free0 - kept
    assert not llm.runners.runner._pending_encodes and c_id not in llm.runners.runner._visual
    llm.exit()


def test_resumable_vision_tower_equals_the_one_piece_tower(tiny):
    arch, weights, _ = tiny
    llm = _llm(weights)
    model = llm.runners.runner.model
    inp = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [1, 2], [_image(11), _image(12, 64)])
    want_main, want_deep = model.encode_vision(inp.pixel_values, inp.image_grid_thw)
    st = model.begin_vision(inp.pixel_values, inp.image_grid_thw)
    assert not model.advance_vision(st, 1) and st.next_block == 1
    assert len(st.deep) == sum(i < 1 for i in arch.vision.deepstack_visual_indexes)  # taps are merged as their block completes
    assert model.advance_vision(st, 5) and st.next_block == 2
    main, deep = model.finish_vision(st)
    assert torch.equal(main, want_main) and len(deep) == len(want_deep) and all(torch.equal(a, b) for a, b in zip(deep, want_deep))
    llm.exit()


def test_pruning_decisions_are_recorded_and_shadow_mode_leaves_the_cache_alone(tiny):
    """A compacting mode records what it kept of every prompt's visual tokens; with ``enable_visual_pruning_shadow`` a
    dense mode records the selection it would have made, drops nothing and generates the dense tokens."""
    arch, weights, oracle = tiny
    tok, proc = load_tokenizer("random:tiny", arch), PatchProcessor(arch)
    inp = prepare_image_inputs(proc, tok, [11, 12, 13], [_image(4)])
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    kw = dict(visual_pruning_keep_ratio=0.5, visual_pruning_min_keep_tokens=8)
    active = _llm(weights, compression_mode="visual_compact_scaled_fp8", **kw)
    active.generate_prepared_image_inputs(inp, sp)
    rec = active.visual_pruning_decisions()
    assert len(rec) == 1 and rec[0]["applied"] and rec[0]["total_visual_tokens"] == 49 and rec[0]["kept"] == 25 and rec[0]["dropped"] == 24
    assert rec[0]["spans"] == [{"modality": "image", "start": 1, "end": 50}] and abs(rec[0]["keep_ratio_actual"] - 25 / 49) < 1e-9
    active.exit()
    shadow = _llm(weights, compression_mode="off", enable_visual_pruning_shadow=True, **kw)
    out = shadow.generate_prepared_image_inputs(inp, sp)
    assert out["token_ids"] == oracle.generate_greedy(inp.input_ids, 4, pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw)
    rec2 = shadow.visual_pruning_decisions(clear=True)
    assert len(rec2) == 1 and not rec2[0]["applied"] and {k: rec2[0][k] for k in ("kept", "dropped", "spans")} == {k: rec[0][k] for k in ("kept", "dropped", "spans")}
    assert shadow.metrics_snapshot()["engine"]["requests"][-1]["dropped_prompt_tokens"] == 0 and shadow.visual_pruning_decisions() == []
    shadow.generate([[5, 6, 7]], sp)                       # text only: nothing to record
    assert shadow.visual_pruning_decisions() == []
    shadow.exit()
    plain = _llm(weights, compression_mode="off")
    plain.generate_prepared_image_inputs(inp, sp)
    assert plain.visual_pruning_decisions() == []          # neither compacting nor shadowing
    plain.exit()


def test_visual_compaction_frees_pages_and_hits(tiny):
    arch, weights, _ = tiny
    img = _image(4)
    llm = _llm(weights, compression_mode="visual_compact_scaled_fp8", visual_pruning_keep_ratio=0.5,
               visual_pruning_min_keep_tokens=8)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    tok = load_tokenizer("random:tiny", arch)
    a = prepare_image_inputs(PatchProcessor(arch), tok, [11, 12, 13], [img])
    b = prepare_image_inputs(PatchProcessor(arch), tok, [31, 32], [img])
    r1 = llm.generate_prepared_image_inputs(a, sp)
    r2 = llm.generate_prepared_image_inputs(b, sp)
    r3 = llm.generate_prepared_image_inputs(a, sp)
    meta = llm.multimodal_prefix_cache_metadata()
    assert meta["hits"] == 2 and meta["resident_tokens"] == 50 - 24  # 49 visual -> 25 kept, + vision_start
    assert r1["token_ids"] == r3["token_ids"]  # cold and hit paths see the same compacted prefix
    assert len(r2["token_ids"]) == 4
    llm.exit()


def test_generate_progress_bar_counts_requests_and_phases(tiny, monkeypatch):
    """``use_tqdm=True`` drives a bar: one update per finished request, prefill and decode
    throughput in the postfix, closed at the end; results are the same with and without it."""
    import io

    from prism_infer_b200.engine import progress as progress_mod
    from prism_infer_b200.engine.contracts import Phase

    class FakeBar:
        instances = []

        def __init__(self, total, **kw):
            self.total, self.n, self.postfixes, self.closed = total, 0, [], False
            FakeBar.instances.append(self)

        def update(self, n):
            self.n += n

        def set_postfix(self, d, refresh=True):
            self.postfixes.append(dict(d))

        def close(self):
            self.closed = True

    real = progress_mod.GenerationProgress
    monkeypatch.setattr("prism_infer_b200.engine.llm_engine.GenerationProgress",
                        lambda total, enabled=True: real(total, enabled=enabled, bar_factory=FakeBar))
    arch, weights, _ = tiny
    llm = _llm(weights)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    prompts = [[1, 2, 3, 4, 5], [7, 8, 9], [11, 12, 13, 14]]
    quiet = llm.generate(prompts, sp, use_tqdm=False)
    assert not FakeBar.instances
    shown = llm.generate(prompts, sp, use_tqdm=True)
    assert [r["token_ids"] for r in shown] == [r["token_ids"] for r in quiet]
    (bar,) = FakeBar.instances
    assert bar.total == 3 and bar.n == 3 and bar.closed
    assert bar.postfixes and set(bar.postfixes[-1]) == {"Prefill", "Decode"}
    assert bar.postfixes[-1]["Decode"].endswith("tok/s") and bar.postfixes[-1]["Decode"] != "0tok/s"
    llm.exit()

    # the reporter on its own: moving averages per phase, plain lines without a bar, tri-state default
    buf = io.StringIO()
    p = real(2, enabled=True, file=buf, bar_factory=lambda **kw: None)
    p.observe_step(Phase.PREFILL, 1000, 0.5)
    p.observe_step(Phase.DECODE, 8, 0.004)
    p.observe_step(Phase.DECODE, 8, 0.008)
    p.observe_step(Phase.IDLE, 0, 0.001)
    assert p.prefill_tok_s == 2000.0 and abs(p.decode_tok_s - (0.7 * 2000 + 0.3 * 1000)) < 1e-6
    p.complete_request()
    p.close()
    assert buf.getvalue().startswith("[1/2] prefill 2000tok/s decode 1700tok/s")
    assert real(1, enabled=None, file=io.StringIO()).enabled is False  # not a terminal: silent


def test_hydrated_vision_result_stays_with_the_sequence(tiny):
    """A burst of submissions larger than the visual-embedding cache: every image is still
    encoded exactly once (the hydrated result is attached to its sequence, not only to the LRU
    cache), nothing is left behind afterwards, and a cancelled request frees its result."""
    arch, weights, oracle = tiny
    llm = _llm(weights, enable_visual_embedding_cache=True, visual_embedding_cache_bytes=1, enable_prefix_caching=False, max_num_seqs=8)
    runner = llm.runners.runner
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)
    reqs = [{"type": "image", "prompt": [3, 4, 5], "image": _image(40 + i, 64)} for i in range(4)]
    outs = llm.generate_mixed(reqs, sp)
    meta = llm.visual_embedding_cache_metadata()
    assert meta["misses"] == 4 and meta["hits"] == 0 and meta["entries"] == 0
    assert not runner._visual and not llm.executor._have_visual
    tok = load_tokenizer("random:tiny", arch)
    inp = prepare_image_inputs(PatchProcessor(arch), tok, [3, 4, 5], [_image(40, 64)])
    assert outs[0]["token_ids"] == oracle.generate_greedy(inp.input_ids, 2, pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw)
    rid = llm.add_vl_request([3, 4, 5], _image(50, 64), sp)
    assert rid in runner._visual
    assert llm.cancel_request(rid) and rid not in runner._visual and not llm.executor._have_visual
    llm.exit()


def test_dense_prefix_is_published_without_an_extra_prefill_step(tiny):
    """A dense multimodal prefix is stored from the chunk that crosses its boundary (one prefill
    step for the whole prompt); only in-place compaction needs the chunk to end on the boundary."""
    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    a = prepare_image_inputs(PatchProcessor(arch), tok, [11, 12, 13], [_image(5)])
    b = prepare_image_inputs(PatchProcessor(arch), tok, [21, 22, 23, 24], [_image(5)])

    def prefill_steps(llm):
        return sum(1 for x in llm.metrics_snapshot()["engine"]["batches"] if x["phase"] == "prefill")

    dense = _llm(weights, compression_mode="scaled_fp8_kv")
    first = dense.generate_prepared_image_inputs(a, sp)
    assert prefill_steps(dense) == 1 and dense.multimodal_prefix_cache_metadata()["stores"] == 1
    second = dense.generate_prepared_image_inputs(b, sp)
    meta = dense.multimodal_prefix_cache_metadata()
    assert meta["hits"] == 1 and prefill_steps(dense) == 2
    assert len(first["token_ids"]) == len(second["token_ids"]) == 3
    dense.exit()
    compact = _llm(weights, compression_mode="visual_compact_scaled_fp8", visual_pruning_keep_ratio=0.5, visual_pruning_min_keep_tokens=4)
    compact.generate_prepared_image_inputs(a, sp)
    assert prefill_steps(compact) == 2 and compact.multimodal_prefix_cache_metadata()["stores"] == 1
    compact.exit()
    off = _llm(weights)  # bf16 dense prefix against the oracle, cold and hit, single prefill step each
    r1 = off.generate_prepared_image_inputs(a, sp)
    r2 = off.generate_prepared_image_inputs(b, sp)
    assert prefill_steps(off) == 2 and off.multimodal_prefix_cache_metadata()["hits"] == 1
    assert r1["token_ids"] == oracle.generate_greedy(a.input_ids, 3, pixel_values=a.pixel_values, image_grid_thw=a.image_grid_thw)
    assert r2["token_ids"] == oracle.generate_greedy(b.input_ids, 3, pixel_values=b.pixel_values, image_grid_thw=b.image_grid_thw)
    off.exit()


def test_vision_jobs_of_one_prefill_step_share_tower_passes(tiny):
    """Five single-image requests prefilled in one step: the tower runs once per microbatch of
    patches, not once per request, and every request still matches the oracle; with the
    embedding cache on, the batched results are stored per request and reused."""
    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    proc = PatchProcessor(arch)
    inputs = [prepare_image_inputs(proc, tok, [30 + i, 31 + i, 32], [_image(60 + i, 64 if i % 2 else 96)]) for i in range(5)]
    want = [oracle.generate_greedy(x.input_ids, 3, pixel_values=x.pixel_values, image_grid_thw=x.image_grid_thw) for x in inputs]

    def run(**kw):
        llm = _llm(weights, max_num_seqs=8, enable_prefix_caching=False, **kw)
        model = llm.runners.runner.model
        calls = []
        real = model.encode_vision
        model.encode_vision = lambda pixels, grids: (calls.append((int(pixels.shape[0]), len(grids))), real(pixels, grids))[1]
        ids = [llm.add_prepared_image_request(x, sp) for x in inputs]
        got = llm._run_until_done(ids)
        return llm, calls, [got[i] for i in ids]

    llm, calls, got = run()
    assert got == want and len(calls) == 1 and calls[0] == (sum(int(x.pixel_values.shape[0]) for x in inputs), 5)
    llm.exit()
    llm, calls, got = run(vision_encoder_microbatch_patches=60, max_vision_patches_per_batch=8192)   # 36- and 16-patch images alternate: two per pass
    assert got == want and len(calls) == 3 and all(p <= 52 for p, _ in calls)
    llm.exit()
    llm, calls, got = run(enable_visual_embedding_cache=True)
    assert got == want
    meta = llm.visual_embedding_cache_metadata()
    assert meta["misses"] == 5 and meta["entries"] == 5 and len(calls) == 5   # hydrated one by one at submission
    again = llm.generate_prepared_image_inputs(inputs[2], sp)
    assert again["token_ids"] == want[2] and llm.visual_embedding_cache_metadata()["hits"] >= 1 and len(calls) == 5
    llm.exit()


@pytest.mark.parametrize("cpu_ratio,counter", [(1.0, "preempt_swap"), (0.0, "preempt_recompute")])
def test_preempted_requests_still_match_the_oracle(tiny, cpu_ratio, counter):
    """Nine pages for three requests that each grow to four: one of them is preempted during
    decode - swapped to CPU pages and back, or dropped and recomputed - and every request still
    produces the oracle's tokens."""
    arch, weights, oracle = tiny
    llm = _llm(weights, num_kvcache_blocks=9, cpu_kv_cache_ratio=cpu_ratio, enable_prefix_caching=False, compression_mode="off")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1000, (20,), generator=g).tolist() for _ in range(3)]
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    assert [o["token_ids"] for o in outs] == [oracle.generate_greedy(p, 40) for p in prompts]
    sched = llm.metrics_snapshot()["scheduler"]
    assert sched[counter] >= 1 and sched["finished"] == 3 and sched["free_gpu_pages"] == 9
    if cpu_ratio:
        assert sched["swap_in"] == sched["preempt_swap"] and sched["free_cpu_pages"] == 9
    llm.exit()


def test_mixed_batch_of_text_image_and_video_matches_the_oracle(tiny):
    """One ``generate_mixed`` call with a text, an image, a two-image and a video request: every
    row equals the oracle run alone (fp32 on CPU is batch-invariant), results keep request order,
    and a per-request ``sampling_params`` overrides the shared one."""
    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    proc = PatchProcessor(arch)
    frames = [_image(70 + i, 64) for i in range(4)]
    img_a, img_b = _image(80, 64), _image(81, 96)
    reqs = [
        {"type": "text", "prompt": [5, 6, 7, 8, 9]},
        {"type": "image", "prompt": [11, 12], "image": img_a},
        {"type": "images", "prompt": [13, 14, 15], "images": [img_a, img_b]},
        {"type": "video", "prompt": [16], "frames": frames, "sampling_params": SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)},
    ]
    llm = _llm(weights, max_num_seqs=8)
    outs = llm.generate_mixed(reqs, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    assert [len(o["token_ids"]) for o in outs] == [5, 5, 5, 2]
    assert outs[0]["token_ids"] == oracle.generate_greedy([5, 6, 7, 8, 9], 5)
    one = prepare_image_inputs(proc, tok, [11, 12], [img_a])
    assert outs[1]["token_ids"] == oracle.generate_greedy(one.input_ids, 5, pixel_values=one.pixel_values, image_grid_thw=one.image_grid_thw)
    two = prepare_image_inputs(proc, tok, [13, 14, 15], [img_a, img_b])
    assert outs[2]["token_ids"] == oracle.generate_greedy(two.input_ids, 5, pixel_values=two.pixel_values, image_grid_thw=two.image_grid_thw)
    vid = prepare_video_inputs(proc, tok, [16], frames)
    assert outs[3]["token_ids"] == oracle.generate_greedy(vid.input_ids, 2, pixel_values=vid.pixel_values, video_grid_thw=vid.video_grid_thw)
    assert all(set(o) == {"text", "raw_text", "token_ids"} and isinstance(o["text"], str) for o in outs)
    with pytest.raises(ValueError, match="unknown request type"):
        llm.generate_mixed([{"type": "audio", "prompt": [1]}], None)
    llm.exit()


def test_output_decoding_and_eos_with_a_scripted_runner():
    """The engine on a runner that returns scripted tokens: generation stops at EOS unless
    ``ignore_eos``; ``text`` drops special tokens, ``raw_text`` keeps them; string prompts go
    through the tokenizer; ``step`` reports signed token counts (prefill +, decode -)."""
    arch = Qwen3VLArch.tiny()
    eos = arch.eos_token_id

    class ScriptedRunners:
        is_driver = True

        def __init__(self, script):
            self.script, self.calls = list(script), []

        def call(self, method, *args):
            self.calls.append(method)
            if method == "execute":
                inp = args[0]
                n = inp.num_seqs if inp.kind == "decode" else len(inp.sample_seq)
                return [self.script.pop(0) for _ in range(n)]
            if method == "capacity":
                return (64, 0)
            return None

        def close(self):
            self.calls.append("close")

    opts = dict(max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64, enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512)
    runners = ScriptedRunners([17, 23, eos, 99, 99])
    llm = LLM("random:tiny", runner_group=runners, device="cpu", **opts)
    out = llm.generate(["12 13 hello"], SamplingParams(temperature=0.0, max_tokens=8))[0]
    assert out["token_ids"] == [17, 23, eos] and out["text"] == "17 23" and out["raw_text"] == f"17 23 {eos}"
    assert runners.script == [99, 99]                               # nothing ran past the EOS
    rid = llm.add_request([5, 6, 7], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    runners.script[:] = [eos, eos]
    done, signed = llm.step()
    assert done == [] and signed == 3                               # prefill of three tokens
    done, signed = llm.step()
    assert signed == -1 and done == [(rid, [eos, eos])]             # EOS ignored: ran to max_tokens
    assert llm.is_finished() and llm.request_state(rid) is None
    llm.exit()
    assert runners.calls[-1] == "close"


def test_device_status_words_are_checked_on_a_cadence():
    """Every ``device_status_check_interval`` steps the engine reads the ranks' status words; a
    set word (here: rank 1 reports a peer wait that ran out) becomes an engine failure."""
    class Runners:
        is_driver = True

        def __init__(self):
            self.status_calls = 0
            self.fail_from = 10 ** 9

        def call(self, method, *args):
            if method == "execute":
                inp = args[0]
                return [7] * (inp.num_seqs if inp.kind == "decode" else len(inp.sample_seq))
            if method == "status":
                self.status_calls += 1
                healthy = {"gemm": (0, 0, 0, 0), "norm": (0, 0, 0, 0)}
                return [healthy, dict(healthy, norm=(2, 5, 17, 3)) if self.status_calls >= self.fail_from else healthy]
            return None

        def close(self):
            pass

    opts = dict(max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64, enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512)
    runners = Runners()
    llm = LLM("random:tiny", runner_group=runners, device="cpu", device_status_check_interval=4, **opts)
    llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    assert runners.status_calls == 2                       # 1 prefill + 8 decode steps
    runners.fail_from = 3
    with pytest.raises(RuntimeError, match="'norm'.: .2, 5, 17, 3"):
        llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    llm.exit()
    quiet = Runners()
    llm = LLM("random:tiny", runner_group=quiet, device="cpu", device_status_check_interval=0, **opts)
    llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    assert quiet.status_calls == 0
    llm.exit()
    with pytest.raises(ValueError):
        LLM("random:tiny", runner_group=Runners(), device="cpu", device_status_check_interval=-1, **opts)


def test_attention_strategy_compacts_by_last_query_scores(tiny, monkeypatch):
    """``visual_pruning_strategy="attention"``: a prompt prefilled in one piece is scored by its
    last query (last decoder layer here), the lowest-scored visual tokens lose their KV rows, the
    rows of the question move down with the prefix, and decoding then equals the oracle with the
    dropped keys masked for generated tokens only (prompt tokens saw everything at prefill)."""
    from prism_infer_b200.models import reference_model

    arch, weights, oracle = tiny
    tok = load_tokenizer("random:tiny", arch)
    inp = prepare_image_inputs(PatchProcessor(arch), tok, [41, 42, 43, 44, 45], [_image(90, 96), _image(91, 64)])
    L = len(inp.input_ids)
    llm = _llm(weights, compression_mode="visual_compact", visual_pruning_strategy="attention", visual_pruning_keep_ratio=0.5,
               visual_pruning_min_keep_tokens=3, visual_pruning_attention_last_n_layers=1, enable_prefix_caching=True)
    layouts, scores_seen = [], []
    commit = llm.executor.bm.commit_compaction
    monkeypatch.setattr(llm.executor.bm, "commit_compaction", lambda seq, plan: (layouts.append(plan.layout), commit(seq, plan))[1])
    take = llm.runners.runner.take_visual_scores
    llm.runners.runner.take_visual_scores = lambda: (lambda s: (scores_seen.append(s), s)[1])(take())
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    got = llm.generate_prepared_image_inputs(inp, sp)["token_ids"]
    assert llm.executor.attention_counters == {"scored": 1, "uniform_fallback": 0}
    (layout,) = layouts
    visual = [i for i, t in enumerate(inp.input_ids) if t == arch.image_token_id]
    kept_visual = [p for p in layout.retained_positions if p in set(visual)]
    assert len(visual) == 13 and len(kept_visual) == 7                       # ceil(13 * 0.5)
    scores = [s for s in scores_seen if s][0]
    (per_token,) = scores.values()
    assert set(per_token) == set(visual) and abs(sum(per_token.values()) - 1.0) < 1.0   # attention mass on visual tokens
    top = sorted(sorted(visual, key=lambda i: (-per_token[i], i))[:7])
    assert kept_visual == top                                                # the highest-scored tokens survive
    boundary = layout.logical_prefix_len
    assert [p for p in layout.retained_positions if p not in set(visual)] == [p for p in range(boundary) if p not in set(visual)]
    assert llm.multimodal_prefix_cache_metadata()["stores"] == 0             # a question-specific prefix is not shared
    llm.exit()

    dropped = torch.tensor(sorted(set(visual) - set(kept_visual)))
    real_sdpa = reference_model.F.scaled_dot_product_attention

    def masked_sdpa(q, k, v, attn_mask=None, is_causal=False, **kw):
        if not is_causal:                       # the vision tower's bidirectional attention
            return real_sdpa(q, k, v, attn_mask=attn_mask, **kw)
        S = q.shape[-2]
        allowed = torch.ones(S, S, dtype=torch.bool).tril()
        if S > L:
            allowed[L:, dropped] = False        # generated tokens do not see the dropped rows
        return real_sdpa(q, k, v, attn_mask=allowed)

    monkeypatch.setattr(reference_model.F, "scaled_dot_product_attention", masked_sdpa)
    want = oracle.generate_greedy(inp.input_ids, 6, pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw)
    monkeypatch.setattr(reference_model.F, "scaled_dot_product_attention", real_sdpa)
    assert got == want
    dense = oracle.generate_greedy(inp.input_ids, 6, pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw)
    assert got[0] == dense[0]                                                 # the first token comes from the uncompacted prefill

    # a prompt that needs several chunks cannot be scored: uniform selection at the prefix boundary
    llm = _llm(weights, compression_mode="visual_compact", visual_pruning_strategy="attention", visual_pruning_keep_ratio=0.5,
               visual_pruning_min_keep_tokens=3, max_chunk_size=16, max_num_batched_tokens=512)
    llm.generate_prepared_image_inputs(inp, sp)
    assert llm.executor.attention_counters == {"scored": 0, "uniform_fallback": 1}
    llm.exit()


@pytest.mark.parametrize("seed,tight", [(3, False), (10, False), (17, False), (5, True), (21, True), (28, True)])
def test_randomised_traffic_with_every_prefill_policy_switched_on(tiny, seed, tight):
    """Cooperative prefill in layer and vision-block quanta, the adaptive (coalescing) policy, the SLO-aware scheduler with
    random deadlines, a small page pool (preemption by swap), random arrivals and random cancellations, all at once: every
    request that was not cancelled gets the oracle's tokens, nothing is left pending and no page leaks.  The tight variant
    has a third of the pages, no coalescing and more heavy images, which brings preemption by swap and SLO interrupts into
    play (seeds chosen so that the six runs together take every branch; another 120 seeds were run once and passed)."""
    import random

    arch, weights, oracle = tiny
    rnd = random.Random(seed)
    tok, proc = load_tokenizer("random:tiny", arch), PatchProcessor(arch)
    now = [1_000_000_000]
    llm = _llm(weights, enable_cooperative_prefill=True, cooperative_prefill_layer_quantum=1, cooperative_prefill_vision_block_quantum=1,
               cooperative_prefill_coalesce_ms=0.0 if tight else 30.0, scheduler_policy="slo_aware", heavy_prefill_vision_patch_threshold=100,
               min_decode_batches_between_heavy_prefills=2, num_kvcache_blocks=13 if tight else 40, cpu_kv_cache_ratio=1.0, max_num_seqs=6,
               max_num_batched_tokens=128, max_chunk_size=64, enable_prefix_caching=True)
    llm.scheduler.clock_ns = lambda: now[0]
    total_pages = llm.scheduler.block_manager.gpu.num_free
    images = [_image(20 + i, 64) for i in range(2)] + [_image(30)]  # two small ones and a heavy one (196 patches)
    plans = []
    for i in range(12):
        n_out = rnd.randint(2, 9)
        if rnd.random() < (0.6 if tight else 0.4):
            img = images[2] if tight and rnd.random() < 0.7 else rnd.choice(images)
            inp = prepare_image_inputs(proc, tok, [rnd.randrange(10, 900) for _ in range(rnd.randint(2, 6))], [img])
            plans.append(("image", inp, n_out))
        else:
            plans.append(("text", [rnd.randrange(10, 900) for _ in range(rnd.randint(3, 90))], n_out))
    arrivals = sorted(rnd.randint(0, 40) for _ in plans)
    submitted, done, cancelled = {}, {}, set()
    step = 0
    while len(submitted) < len(plans) or not llm.is_finished():
        while len(submitted) < len(plans) and arrivals[len(submitted)] <= step:
            kind, payload, n_out = plans[len(submitted)]
            sp = SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True)
            rid = llm.add_prepared_image_request(payload, sp) if kind == "image" else llm.add_request(payload, sp)
            seq = llm._sequences[rid]
            seq.arrival_ns = now[0]
            if rnd.random() < 0.5:
                seq.deadline_ns = now[0] + rnd.choice([50, 200, 900]) * 1_000_000
            submitted[rid] = (kind, payload, n_out)
        if submitted and rnd.random() < 0.06:
            victim = rnd.choice(list(submitted))
            if victim not in done and victim not in cancelled and llm.cancel_request(victim):
                cancelled.add(victim)
        for o in llm.step_result().outputs:
            if o.finished:
                done[o.request_id] = list(o.token_ids)
        now[0] += 7_000_000  # seven milliseconds per engine step
        step += 1
        assert step < 3000, "the engine stopped making progress"
    assert llm._pending_prefill is None and llm._pending_vision is None and not llm._deferred
    assert set(done) | cancelled >= set(submitted) and len(submitted) == len(plans)
    for rid, (kind, payload, n_out) in submitted.items():
        if rid in cancelled and rid not in done:
            continue
        # the oracle recomputes the whole sequence per token and takes every placeholder id for a visual row, so it can
        # only follow a generation up to (and including) a placeholder id that the random model happened to emit
        got = done[rid]
        stop = next((i + 1 for i, t in enumerate(got) if t in (arch.image_token_id, arch.video_token_id)), len(got))
        assert len(got) == n_out
        want = oracle.generate_greedy(payload.input_ids, stop, pixel_values=payload.pixel_values, image_grid_thw=payload.image_grid_thw) \
            if kind == "image" else oracle.generate_greedy(payload, stop)
        assert got[:stop] == want, (rid, kind, n_out)
    kept = llm.multimodal_prefix_cache_metadata()["resident_pages"]
    assert llm.scheduler.block_manager.gpu.num_free == total_pages - kept
    assert not llm.runners.runner.__dict__.get("_pending_encodes") and not llm.runners.runner.__dict__.get("_pending_prefills")
    llm.exit()


def test_image_requests_accept_file_paths(tiny, tmp_path):
    from PIL import Image

    arch, weights, _ = tiny
    arr = _image(13, 64)
    path = tmp_path / "picture.png"
    Image.fromarray(arr).save(path)
    llm = _llm(weights)
    sp = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    assert llm.generate_images([5, 6], [str(path)], sp)["token_ids"] == llm.generate_images([5, 6], [arr], sp)["token_ids"]
    assert llm.generate_images([5, 6], [path], sp)["token_ids"] == llm.generate_images([5, 6], [Image.fromarray(arr)], sp)["token_ids"]
    llm.exit()
