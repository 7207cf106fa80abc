"""Arrival loop and media caches with a fake clock on the tiny CPU engine."""

import numpy as np
import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.engine.online import OnlineRequest, OnlineServingSession, media_fingerprint
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.weights import random_weights


class FakeClock:
    def __init__(self):
        self.t = 0

    def now(self):
        self.t += 200_000  # every look at the clock costs 0.2 ms
        return self.t

    def sleep(self, s):
        self.t += int(max(s, 0.0) * 1e9)


@pytest.fixture(scope="module")
def engine():
    arch = Qwen3VLArch.tiny()
    llm = LLM("random:tiny", weights=random_weights(arch, dtype=torch.float32, seed=0), device="cpu", max_model_len=512,
              kvcache_block_size=16, num_kvcache_blocks=96, enforce_eager=True, max_chunk_size=256)
    yield llm
    llm.exit()


def _img(seed):
    return np.random.default_rng(seed).integers(0, 256, (64, 64, 3), dtype=np.uint8)


def test_fingerprint_is_content_addressed():
    a, b = _img(1), _img(1).copy()
    assert media_fingerprint(a) == media_fingerprint(b) != media_fingerprint(_img(2))
    assert media_fingerprint(torch.from_numpy(a)) != media_fingerprint(a)  # typed, not just bytes
    assert media_fingerprint([a, b]) == media_fingerprint((a, b))


def test_online_run_arrivals_caches_and_cancellation(engine):
    clock = FakeClock()
    session = OnlineServingSession(engine, clock_ns=clock.now, sleep=clock.sleep, background_preprocessing=False)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    img = _img(5)
    reqs = [
        OnlineRequest("t0", 0.0, {"type": "text", "prompt": [1, 2, 3]}, sp),
        OnlineRequest("i0", 0.010, {"type": "image", "prompt": "11 12", "image": img}, sp),
        OnlineRequest("i1", 0.020, {"type": "image", "prompt": "21 22 23", "image": img.copy()}, sp, ttft_slo_ms=500.0),
        OnlineRequest("m0", 0.030, {"type": "interleaved_images", "prompt": "7 <image> 8 <image> 9 10",
                                    "images": [img, _img(6)]}, sp),
        OnlineRequest("c0", 0.040, {"type": "text", "prompt": list(range(50))},
                      SamplingParams(temperature=0.0, max_tokens=400, ignore_eos=True), cancel_offset_s=0.041),
    ]
    out = session.run(reqs)
    by = {r.request_key: r for r in out.requests}
    assert [r.request_key for r in out.requests] == ["t0", "i0", "i1", "m0", "c0"]
    for k in ("t0", "i0", "i1", "m0"):
        assert by[k].finish_reason == "length" and len(by[k].token_ids) == 4
        assert by[k].ttft_ms is not None and by[k].latency_ms >= by[k].ttft_ms
    assert by["c0"].finish_reason == "cancelled" and len(by["c0"].token_ids) < 400
    # same pixels, new question: processor + layout cache hit, prompt rebound, prefix KV reused
    assert out.cache_counters["processor_hits"] >= 2 and out.cache_counters["rebinds"] >= 1
    assert by["i1"].cached_tokens == 1 + 4 and by["i0"].cached_tokens == 0  # vision_start + 2x2 merged tokens
    assert out.duration_s > 0.04 and out.steps > 0
    rec = out.to_record()
    assert len(rec["requests"]) == 5
    session.close()


def test_online_request_validation():
    sp = SamplingParams()
    with pytest.raises(ValueError):
        OnlineRequest("", 0.0, {"type": "text", "prompt": "x"}, sp)
    with pytest.raises(ValueError):
        OnlineRequest("a", -1.0, {"type": "text", "prompt": "x"}, sp)
    with pytest.raises(ValueError):
        OnlineRequest("a", 1.0, {"type": "audio", "prompt": "x"}, sp)
    with pytest.raises(ValueError):
        OnlineRequest("a", 1.0, {"type": "text", "prompt": "x"}, sp, cancel_offset_s=0.5)
