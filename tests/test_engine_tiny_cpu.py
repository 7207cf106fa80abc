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
