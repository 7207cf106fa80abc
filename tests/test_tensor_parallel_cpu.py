"""Tensor-parallel host logic on CPU ranks (gloo): spawned workers, shared-memory control
plane, sharded weights, vocabulary-parallel embedding / LM head, lock-step KV commands."""

import numpy as np
import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.reference_model import ReferenceQwen3VL
from prism_infer_b200.models.weights import random_weights
from prism_infer_b200.utils.tokenizer import load_tokenizer

pytestmark = pytest.mark.distributed


@pytest.mark.timeout(300)
def test_tp2_cpu_matches_oracle_and_prefix_cache_works():
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    oracle = ReferenceQwen3VL(arch, weights)
    llm = LLM("random:tiny", weights=weights, tensor_parallel_size=2, max_model_len=512, kvcache_block_size=16,
              num_kvcache_blocks=64, enforce_eager=True, max_chunk_size=64, tensor_parallel_timeout_seconds=120)
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
        prompts = [[5, 6, 7, 8, 9], list(range(100, 140))]
        outs = llm.generate(prompts, sp)
        for p, o in zip(prompts, outs):
            assert o["token_ids"] == oracle.generate_greedy(p, 6)
        img = np.random.default_rng(0).integers(0, 256, (64, 64, 3), dtype=np.uint8)
        tok = load_tokenizer("random:tiny", arch)
        a = prepare_image_inputs(PatchProcessor(arch), tok, [11, 12, 13], [img])
        b = prepare_image_inputs(PatchProcessor(arch), tok, [21, 22], [img])
        ra = llm.generate_prepared_image_inputs(a, sp)
        rb = llm.generate_prepared_image_inputs(b, sp)  # prefix hit: copy_prefix runs on both ranks
        assert llm.multimodal_prefix_cache_metadata()["hits"] == 1
        assert ra["token_ids"] == oracle.generate_greedy(a.input_ids, 6, pixel_values=a.pixel_values, image_grid_thw=a.image_grid_thw)
        assert rb["token_ids"] == oracle.generate_greedy(b.input_ids, 6, pixel_values=b.pixel_values, image_grid_thw=b.image_grid_thw)
    finally:
        llm.exit()


@pytest.mark.timeout(300)
def test_tp2_cpu_attention_strategy_scores_are_reduced_over_ranks():
    """Each rank scores with its own heads; after the reduction both compact the same rows, so
    the two-rank engine produces the single-rank engine's tokens."""
    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    tok = load_tokenizer("random:tiny", arch)
    rng = np.random.default_rng(3)
    inp = prepare_image_inputs(PatchProcessor(arch), tok, [41, 42, 43, 44], [rng.integers(0, 256, (96, 96, 3), dtype=np.uint8)])
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    opts = dict(max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64, enforce_eager=True, max_chunk_size=256,
                compression_mode="visual_compact", visual_pruning_strategy="attention", visual_pruning_keep_ratio=0.5,
                visual_pruning_min_keep_tokens=2)
    one = LLM("random:tiny", weights=weights, device="cpu", **opts)
    want = one.generate_prepared_image_inputs(inp, sp)["token_ids"]
    assert one.executor.attention_counters["scored"] == 1
    one.exit()
    two = LLM("random:tiny", weights=weights, tensor_parallel_size=2, tensor_parallel_timeout_seconds=120, **opts)
    try:
        got = two.generate_prepared_image_inputs(inp, sp)["token_ids"]
        assert two.executor.attention_counters["scored"] == 1
    finally:
        two.exit()
    assert got == want


@pytest.mark.timeout(300)
def test_tp2_cpu_loads_an_upstream_checkpoint_directory_and_matches_upstream_tokens(tmp_path):
    """What a deployment does: a checkpoint directory written by the upstream ``save_pretrained`` (several safetensors
    shards with an index), two ranks that each read their own slices of it, and the tokens of the upstream model."""
    hf = pytest.importorskip("transformers.models.qwen3_vl")
    arch = Qwen3VLArch.tiny()
    torch.manual_seed(0)
    model = hf.Qwen3VLForConditionalGeneration(hf.Qwen3VLConfig(**arch.to_hf_config())).eval().float()
    g = torch.Generator().manual_seed(3)
    model.load_state_dict({k: torch.randn(v.shape, generator=g) * (0.05 if v.ndim > 1 else 0.2) + (1.0 if ("norm" in k and k.endswith("weight")) else 0.0)
                           for k, v in model.state_dict().items()})
    model.save_pretrained(tmp_path / "ckpt", safe_serialization=True, max_shard_size="400KB")
    img = np.random.default_rng(1).integers(0, 256, (64, 96, 3), dtype=np.uint8)
    inp = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [9, 8, 7], [img])

    def upstream_next(extra):
        ids = torch.tensor([list(inp.input_ids) + extra])
        mm = torch.zeros_like(ids, dtype=torch.int32)
        mm[ids == arch.image_token_id] = 1
        with torch.no_grad():
            out = model(input_ids=ids, attention_mask=torch.ones_like(ids), mm_token_type_ids=mm, pixel_values=inp.pixel_values.float(),
                        image_grid_thw=torch.tensor(inp.image_grid_thw))
        return int(torch.argmax(out.logits[0, -1]))

    want = []
    for _ in range(5):
        want.append(upstream_next(want))
    llm = LLM(str(tmp_path / "ckpt"), tensor_parallel_size=2, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=32,
              enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256, tensor_parallel_timeout_seconds=120)
    try:
        got = llm.generate_prepared_image_inputs(inp, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))["token_ids"]
    finally:
        llm.exit()
    assert got == want


@pytest.mark.timeout(300)
def test_tp2_cpu_worker_killed_in_mid_stream_is_replaced_and_the_stream_continues():
    """Recovery from a lost rank, end to end on two CPU ranks: the serving runtime streams a greedy request from a
    two-rank engine, the worker process is killed between tokens (a host-side fault), the driver names the dead rank
    with its exit code without waiting for the command deadline, the runtime builds a new two-rank engine and the
    client's stream continues; all tokens equal the oracle's and none arrives twice."""
    import os
    import signal

    from prism_infer_b200.serving import EventKind, GenerationRequest, Modality, ServingRuntime

    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    built = []

    def make():
        built.append(LLM("random:tiny", weights=weights, tensor_parallel_size=2, max_model_len=256, kvcache_block_size=16,
                         num_kvcache_blocks=64, enforce_eager=True, max_chunk_size=64, tensor_parallel_timeout_seconds=60))
        return built[-1]

    rt = ServingRuntime(make, max_restarts=1)
    rt.start()
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
        handle = rt.submit(GenerationRequest("r", "5 6 7 8 9", Modality.TEXT, None, sp))
        tokens, final = [], None
        while final is None:
            ev = handle.next_event_blocking(120.0)
            if ev.kind is EventKind.TOKEN:
                tokens.append(ev.token_id)
                if len(tokens) == 3:
                    os.kill(built[0].runners.procs[0].pid, signal.SIGKILL)
            elif ev.kind in (EventKind.DONE, EventKind.ERROR):
                final = ev
        assert final.kind is EventKind.DONE, final.error
        assert tokens == list(final.token_ids) == ReferenceQwen3VL(arch, weights).generate_greedy([5, 6, 7, 8, 9], 24)
        assert len(built) == 2 and len(rt.restarts) == 1 and rt.is_healthy
        assert "TPWorkerExited" in rt.restarts[0] and "{1: -9}" in rt.restarts[0]
    finally:
        rt.stop()
