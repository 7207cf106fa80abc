"""Serving runtime and HTTP app against a fake engine that implements only the
``ServingEngine`` protocol (the reference's strategy, tests/test_serving_runtime.py:28-114)."""

import asyncio
import base64
import io
import json
import threading
import time

import httpx
import pytest

from prism_infer_b200.engine.contracts import Phase, RequestOutput, StepResult
from prism_infer_b200.engine.request import RequestState
from prism_infer_b200.sampling_params import SamplingParams
from prism_infer_b200.serving import (DuplicateRequest, EventKind, GenerationRequest, IngressFull, Modality,
                                      RuntimeUnavailable, ServingRuntime)
from prism_infer_b200.serving.app import create_app
from prism_infer_b200.serving.cli import load_engine_options


class FakeTokenizer:
    def decode(self, ids, skip_special_tokens=True):
        return " ".join(f"t{i}" for i in ids)


class FakeEngine:
    """Emits tokens 100, 101, ... per request, one per step, up to max_tokens."""

    def __init__(self, fail_after=None, step_delay=0.0):
        self.tokenizer = FakeTokenizer()
        self.live = {}
        self.next_id = 0
        self.fail_after = fail_after
        self.steps = 0
        self.step_delay = step_delay
        self.cancelled = []
        self.exited = False
        self.media_seen = []

    def _add(self, prompt, sp, media=None, raise_on_reject=True):
        if prompt == "reject me":
            eid = self.next_id
            self.next_id += 1
            self.live[eid] = None
            return eid
        eid = self.next_id
        self.next_id += 1
        self.live[eid] = [sp.max_tokens, 0]
        self.media_seen.append(media)
        return eid

    def add_request(self, prompt, sampling_params=None, *, raise_on_reject=True):
        return self._add(prompt, sampling_params, None, raise_on_reject)

    def add_vl_request(self, prompt, image, sampling_params=None, **kw):
        return self._add(prompt, sampling_params, ("image", image))

    def add_images_request(self, prompt, images, sampling_params=None, **kw):
        return self._add(prompt, sampling_params, ("images", len(images)))

    def add_video_request(self, prompt, frames, sampling_params=None, **kw):
        return self._add(prompt, sampling_params, ("video", len(frames)))

    def request_state(self, eid):
        if self.live.get(eid, 0) is None:
            del self.live[eid]
            return RequestState.REJECTED
        return RequestState.WAITING

    def is_finished(self):
        return not self.live

    def cancel_request(self, eid):
        self.cancelled.append(eid)
        return self.live.pop(eid, None) is not None

    def step_result(self):
        self.steps += 1
        if self.fail_after is not None and self.steps > self.fail_after:
            raise RuntimeError("boom")
        if self.step_delay:
            time.sleep(self.step_delay)
        outs = []
        for eid, st in list(self.live.items()):
            st[1] += 1
            done = st[1] >= st[0]
            outs.append(RequestOutput(eid, 100 + st[1], done, "length" if done else None))
            if done:
                del self.live[eid]
        return StepResult(Phase.DECODE, tuple(outs), len(outs))

    def exit(self):
        self.exited = True


def _req(rid, prompt="hello", max_tokens=3, modality=Modality.TEXT, media=None):
    return GenerationRequest(rid, prompt, modality, media, SamplingParams(temperature=0.0, max_tokens=max_tokens))


def _drain(handle, timeout=5.0):
    events = []
    while True:
        ev = handle.next_event_blocking(timeout)
        events.append(ev)
        if ev.kind in (EventKind.DONE, EventKind.ERROR):
            return events


def test_runtime_streams_tokens_then_done_and_shuts_down():
    eng = FakeEngine()
    rt = ServingRuntime(lambda: eng, ingress_capacity=4)
    rt.start()
    assert rt.is_healthy
    events = _drain(rt.submit(_req("a", max_tokens=3)))
    kinds = [e.kind for e in events]
    assert kinds == [EventKind.ACCEPTED, EventKind.TOKEN, EventKind.TOKEN, EventKind.TOKEN, EventKind.DONE]
    assert [e.token_id for e in events[1:4]] == [101, 102, 103]
    assert events[1].token_text == "t101"
    done = events[-1]
    assert done.token_ids == (101, 102, 103) and done.text == "t101 t102 t103" and done.finish_reason == "length"
    assert done.to_dict()["token_ids"] == [101, 102, 103]
    rejected = _drain(rt.submit(_req("r", prompt="reject me")))
    assert rejected[-1].kind is EventKind.DONE and rejected[-1].finish_reason == "rejected"
    rt.stop()
    assert eng.exited and not rt.is_healthy


def test_runtime_backpressure_duplicates_and_cancellation():
    eng = FakeEngine(step_delay=0.02)
    rt = ServingRuntime(lambda: eng, ingress_capacity=64)
    rt.start()
    h = rt.submit(_req("long", max_tokens=10_000))
    with pytest.raises(DuplicateRequest):
        rt.submit(_req("long"))
    first = h.next_event_blocking(5.0)
    assert first.kind is EventKind.ACCEPTED
    rt.cancel("long")
    events = _drain(h)
    assert events[-1].kind is EventKind.DONE and events[-1].finish_reason == "cancelled"
    assert eng.cancelled == [first.engine_request_id]
    rt.stop()
    # a stalled owner thread makes the bounded ingress overflow
    gate = threading.Event()

    class Stalled(FakeEngine):
        def is_finished(self):
            gate.wait(5.0)
            return super().is_finished()

    rt2 = ServingRuntime(lambda: Stalled(), ingress_capacity=2)
    rt2.start()
    time.sleep(0.05)
    rt2.submit(_req("x1"))
    rt2.submit(_req("x2"))
    with pytest.raises(IngressFull):
        for i in range(3, 8):
            rt2.submit(_req(f"x{i}"))
    gate.set()
    rt2.stop()


def test_engine_failure_reaches_every_request_and_health():
    eng = FakeEngine(fail_after=2)
    rt = ServingRuntime(lambda: eng)
    rt.start()
    h1, h2 = rt.submit(_req("a", max_tokens=50)), rt.submit(_req("b", max_tokens=50))
    for h in (h1, h2):
        events = _drain(h)
        assert events[-1].kind is EventKind.ERROR and "boom" in events[-1].error
    time.sleep(0.05)
    assert not rt.is_healthy and isinstance(rt.failure, RuntimeError)
    rt.stop()


def test_restart_replays_greedy_requests_without_repeating_tokens():
    """With ``max_restarts`` a failed step costs the clients nothing they can see: the engine is rebuilt, open greedy
    requests run again from their prompts, tokens already delivered are checked and not sent twice, and a request that
    samples ends with an error.  A second failure beyond the allowance ends the runtime as without the option."""
    built = []

    def factory():
        built.append(FakeEngine(fail_after=3 if not built else None))
        return built[-1]

    rt = ServingRuntime(factory, max_restarts=1)
    rt.start()
    greedy = [rt.submit(_req(f"g{i}", max_tokens=8)) for i in range(2)]
    sampled = rt.submit(GenerationRequest("s", "hello", Modality.TEXT, None, SamplingParams(temperature=0.8, max_tokens=8)))
    for h in greedy:
        events = _drain(h)
        assert [e.kind for e in events].count(EventKind.ACCEPTED) == 1
        assert [e.token_id for e in events if e.kind is EventKind.TOKEN] == list(range(101, 109))
        assert events[-1].kind is EventKind.DONE and events[-1].token_ids == tuple(range(101, 109))
    events = _drain(sampled)
    assert events[-1].kind is EventKind.ERROR and "sampled" in events[-1].error
    assert rt.is_healthy and len(built) == 2 and built[0].exited and len(rt.restarts) == 1 and "boom" in rt.restarts[0]
    # a request after the restart is served by the new engine
    assert _drain(rt.submit(_req("after", max_tokens=2)))[-1].token_ids == (101, 102)
    rt.stop()

    # the new engine answers differently: the request ends with an error instead of a stream that changes its mind
    class Shifted(FakeEngine):
        def step_result(self):
            res = super().step_result()
            return StepResult(res.phase, tuple(RequestOutput(o.request_id, o.new_token + 1000, o.finished, o.finish_reason)
                                               for o in res.outputs), res.num_tokens)

    built2 = []

    def factory2():
        built2.append(FakeEngine(fail_after=2) if not built2 else Shifted())
        return built2[-1]

    rt2 = ServingRuntime(factory2, max_restarts=1)
    rt2.start()
    events = _drain(rt2.submit(_req("x", max_tokens=8)))
    assert events[-1].kind is EventKind.ERROR and "did not reproduce" in events[-1].error and built2[1].cancelled
    rt2.stop()

    # the allowance is spent: the next failure is final
    built3 = []

    def factory3():
        built3.append(FakeEngine(fail_after=2))
        return built3[-1]

    rt3 = ServingRuntime(factory3, max_restarts=1)
    rt3.start()
    events = _drain(rt3.submit(_req("y", max_tokens=50)))
    assert events[-1].kind is EventKind.ERROR and "boom" in events[-1].error
    time.sleep(0.05)
    assert not rt3.is_healthy and len(built3) == 2
    rt3.stop()


def test_shutdown_finishes_open_requests():
    eng = FakeEngine(step_delay=0.01)
    rt = ServingRuntime(lambda: eng)
    rt.start()
    h = rt.submit(_req("s", max_tokens=100_000))
    assert h.next_event_blocking(5.0).kind is EventKind.ACCEPTED
    rt.stop()
    events = _drain(h)
    assert events[-1].finish_reason == "shutdown"


def _png_data_url():
    from PIL import Image

    buf = io.BytesIO()
    Image.new("RGB", (32, 32), (10, 20, 30)).save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def test_http_app_json_sse_and_status_codes():
    eng = FakeEngine()
    rt = ServingRuntime(lambda: eng, ingress_capacity=8)
    rt.start()
    app = create_app(rt, manage_runtime=False)

    async def scenario():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as client:
            assert (await client.get("/health")).json() == {"status": "ok"}
            r = await client.post("/v1/generate", json={"prompt": "hi", "sampling": {"max_tokens": 2}})
            assert r.status_code == 200
            body = r.json()
            assert body["event"] == "done" and body["token_ids"] == [101, 102] and body["finish_reason"] == "length"
            # unknown field -> 422 from the strict schema; inconsistent media -> 422
            assert (await client.post("/v1/generate", json={"prompt": "hi", "bogus": 1})).status_code == 422
            assert (await client.post("/v1/generate", json={"prompt": "hi", "modality": "image"})).status_code == 422
            # image and video bodies reach the right engine entry points
            url = _png_data_url()
            r = await client.post("/v1/generate", json={"prompt": "what", "modality": "image", "media": url,
                                                         "sampling": {"max_tokens": 1}})
            assert r.status_code == 200
            r = await client.post("/v1/generate", json={"prompt": "what", "modality": "video", "media": [url, url],
                                                         "sampling": {"max_tokens": 1}})
            assert r.status_code == 200
            r = await client.post("/v1/generate", json={"prompt": "x", "modality": "image", "media": "data:image/png;base64,@@"})
            assert r.status_code == 400
            # SSE stream
            async with client.stream("POST", "/v1/generate", json={"prompt": "hi", "stream": True, "request_id": "sse-1",
                                                                  "sampling": {"max_tokens": 2}}) as resp:
                text = (await resp.aread()).decode()
            frames = [f for f in text.split("\n\n") if f]
            assert [f.split("\n")[0] for f in frames] == ["event: accepted", "event: token", "event: token", "event: done"]
            assert json.loads(frames[-1].split("data: ", 1)[1])["token_ids"] == [101, 102]

    asyncio.run(scenario())
    assert eng.media_seen[-3][0] == "image" and eng.media_seen[-2] == ("video", 2)
    rt.stop()

    async def down():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t") as client:
            assert (await client.get("/health")).status_code == 503
            assert (await client.post("/v1/generate", json={"prompt": "hi"})).status_code == 503

    asyncio.run(down())


def test_openai_style_chat_completions():
    """``/v1/chat/completions`` and ``/v1/models`` over the fake engine: a plain answer, a streamed one ending with
    ``[DONE]``, a user turn with text and image parts (one image -> single-image request, two -> multi-image), a system
    message put before the user's text, fields a client adds being ignored, and 400 for conversations of several turns
    and for unknown part types."""
    eng = FakeEngine()
    seen = []
    inner = eng._add

    def spy(prompt, sp, media=None, raise_on_reject=True):
        seen.append((prompt, sp.max_tokens, sp.temperature))
        return inner(prompt, sp, media, raise_on_reject)

    eng._add = spy
    rt = ServingRuntime(lambda: eng, ingress_capacity=8)
    rt.start()
    app = create_app(rt, manage_runtime=False, model_name="tiny-vl")
    url = _png_data_url()

    async def scenario():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t") as c:
            assert (await c.get("/v1/models")).json()["data"][0]["id"] == "tiny-vl"
            r = await c.post("/v1/chat/completions", json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                                          "top_p": 0.9, "user": "someone"})
            body = r.json()
            assert r.status_code == 200 and body["object"] == "chat.completion" and body["model"] == "m" and body["id"].startswith("chatcmpl-")
            assert body["choices"] == [{"index": 0, "message": {"role": "assistant", "content": "t101 t102 t103"}, "finish_reason": "length"}]
            assert body["usage"] == {"completion_tokens": 3} and seen[-1] == ("hi", 3, 0.0)
            async with c.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "system", "content": "Be brief."},
                                {"role": "user", "content": "hi"}], "max_completion_tokens": 2, "stream": True}) as resp:
                frames = [f[len("data: "):] for f in (await resp.aread()).decode().split("\n\n") if f]
            assert frames[-1] == "[DONE]" and seen[-1] == ("Be brief.\n\nhi", 2, 0.0)
            chunks = [json.loads(f) for f in frames[:-1]]
            assert all(ch["object"] == "chat.completion.chunk" and ch["model"] == "tiny-vl" for ch in chunks)
            assert [ch["choices"][0]["delta"] for ch in chunks] == [{"role": "assistant", "content": ""}, {"content": "t101"}, {"content": "t102"}, {}]
            assert [ch["choices"][0]["finish_reason"] for ch in chunks] == [None, None, None, "length"]
            one = {"role": "user", "content": [{"type": "text", "text": "what is this?"}, {"type": "image_url", "image_url": {"url": url}}]}
            assert (await c.post("/v1/chat/completions", json={"messages": [one], "max_tokens": 1})).status_code == 200
            assert eng.media_seen[-1][0] == "image" and seen[-1][0] == "what is this?"
            two = {"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}, {"type": "image_url", "image_url": url},
                                               {"type": "text", "text": "compare"}]}
            assert (await c.post("/v1/chat/completions", json={"messages": [two], "max_tokens": 1})).status_code == 200
            assert eng.media_seen[-1] == ("images", 2)
            turns = [{"role": "user", "content": "a"}, {"role": "assistant", "content": "b"}, {"role": "user", "content": "c"}]
            r = await c.post("/v1/chat/completions", json={"messages": turns})
            assert r.status_code == 400 and "several turns" in r.json()["detail"]
            bad = {"role": "user", "content": [{"type": "input_audio", "input_audio": {}}]}
            assert (await c.post("/v1/chat/completions", json={"messages": [bad]})).status_code == 400
            assert (await c.post("/v1/chat/completions", json={"messages": []})).status_code == 422

    try:
        asyncio.run(scenario())
    finally:
        rt.stop()


def test_first_token_target_reaches_the_engine():
    """``ttft_slo_ms`` of ``/v1/generate`` becomes the request's deadline in the engine (arrival + target), which the
    SLO-aware scheduler policy orders by; nonsense values are refused by the schema and by the request type."""
    import torch

    from prism_infer_b200 import LLM
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    weights = random_weights(Qwen3VLArch.tiny(), dtype=torch.float32, seed=0)
    seen = {}

    def make():
        eng = LLM("random:tiny", weights=weights, device="cpu", max_model_len=128, kvcache_block_size=16, num_kvcache_blocks=32,
                  enforce_eager=True, scheduler_policy="slo_aware")
        inner = eng.set_first_token_deadline

        def spy(rid, ms):
            ok = inner(rid, ms)
            if ok:
                seq = eng._sequences[rid]
                seen[rid] = (ms, seq.deadline_ns - seq.arrival_ns)
            return ok

        eng.set_first_token_deadline = spy
        return eng

    rt = ServingRuntime(make)
    rt.start()
    app = create_app(rt, manage_runtime=False)

    async def scenario():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t", timeout=60.0) as c:
            body = {"prompt": "7 8 9", "sampling": {"max_tokens": 2, "ignore_eos": True}}
            r = await c.post("/v1/generate", json={**body, "ttft_slo_ms": 250})
            assert r.status_code == 200 and len(r.json()["token_ids"]) == 2
            assert (await c.post("/v1/generate", json=body)).status_code == 200  # no target: the engine is not asked
            for bad in (0, -5, "soon"):
                assert (await c.post("/v1/generate", json={**body, "ttft_slo_ms": bad})).status_code == 422

    try:
        asyncio.run(scenario())
        assert list(seen.values()) == [(250.0, 250_000_000)]
        assert rt.engine.set_first_token_deadline(10_000, 5.0) is False
        with pytest.raises(ValueError):
            GenerationRequest("x", "hi", Modality.TEXT, None, SamplingParams(), ttft_slo_ms=float("inf"))
        with pytest.raises(ValueError):
            rt.engine.set_first_token_deadline(0, float("nan"))
    finally:
        rt.stop()


def test_cancel_endpoint_and_cancellation_before_admission():
    """``DELETE /v1/requests/{id}`` ends an open request with ``cancelled`` (404 for an unknown id), and a cancellation
    that overtakes its request in the ingress queue still takes effect when the request is taken out."""
    eng = FakeEngine(step_delay=0.005)
    rt = ServingRuntime(lambda: eng, ingress_capacity=8)
    rt.start()
    app = create_app(rt, manage_runtime=False)

    async def scenario():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t", timeout=30.0) as c:
            assert (await c.delete("/v1/requests/nobody")).status_code == 404
            pending = asyncio.ensure_future(c.post("/v1/generate", json={"request_id": "long", "prompt": "hi", "sampling": {"max_tokens": 100000}}))
            while not rt.is_open("long"):
                await asyncio.sleep(0.01)
            r = await c.delete("/v1/requests/long")
            assert r.status_code == 202 and r.json() == {"request_id": "long", "status": "cancelling"}
            answer = await pending
            assert answer.status_code == 200 and answer.json()["finish_reason"] == "cancelled"
            assert not rt.is_open("long") and (await c.delete("/v1/requests/long")).status_code == 404

    try:
        asyncio.run(scenario())
    finally:
        rt.stop()

    # the cancellation is consumed before the request is admitted: the owner thread remembers it
    gate = threading.Event()

    class Gated(FakeEngine):
        def is_finished(self):
            gate.wait(5.0)
            return super().is_finished()

    eng2 = Gated()
    rt2 = ServingRuntime(lambda: eng2, ingress_capacity=8)
    rt2.start()
    try:
        time.sleep(0.05)             # the owner thread now waits inside is_finished, past its cancellation check
        h = rt2.submit(_req("early", max_tokens=50))
        rt2.cancel("early")
        gate.set()
        events = _drain(h)
        assert events[-1].finish_reason == "cancelled" and events[-1].token_ids == () and eng2.next_id == 0  # never reached the engine
    finally:
        gate.set()
        rt2.stop()


def test_cli_engine_config(tmp_path):
    p = tmp_path / "cfg.json"
    p.write_text(json.dumps({"tensor_parallel_size": 2, "max_model_len": 512}))
    assert load_engine_options(str(p)) == {"tensor_parallel_size": 2, "max_model_len": 512}
    p.write_text(json.dumps({"model": "x"}))
    with pytest.raises(ValueError):
        load_engine_options(str(p))
    assert load_engine_options(None) == {}


def test_http_server_with_the_real_engine_on_cpu():
    """The whole stack without a fake: tiny random-weight engine on CPU behind the runtime and the HTTP app.  A text
    request as JSON, an image request as an SSE stream and three concurrent text requests; the tokens are the ones the
    engine gives when it is driven directly, and an image request equals the oracle."""
    import base64
    import io

    import numpy as np
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.reference_model import ReferenceQwen3VL
    from prism_infer_b200.models.weights import random_weights

    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)

    def make():
        return LLM("random:tiny", weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=64,
                   enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256, max_num_seqs=4)

    direct = make()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    want_text = {p: direct.generate([p], sp)[0]["token_ids"] for p in ("7 8 9", "10 11", "12 13 14 15")}
    arr = np.random.default_rng(3).integers(0, 256, (64, 64, 3), dtype=np.uint8)
    want_image = direct.generate_images("21 22", [Image.fromarray(arr)], sp)["token_ids"]
    inputs = direct.prepare_images("21 22", [Image.fromarray(arr)])
    assert want_image == ReferenceQwen3VL(arch, weights).generate_greedy(inputs.input_ids, 5, pixel_values=inputs.pixel_values,
                                                                        image_grid_thw=inputs.image_grid_thw)
    direct.exit()
    buf = io.BytesIO()
    Image.fromarray(arr).save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()

    rt = ServingRuntime(make, ingress_capacity=8)
    rt.start()
    app = create_app(rt, manage_runtime=False)

    async def scenario():
        transport = httpx.ASGITransport(app=app)
        async with httpx.AsyncClient(transport=transport, base_url="http://t", timeout=60.0) as client:
            body = {"sampling": {"max_tokens": 5, "ignore_eos": True}}
            r = await client.post("/v1/generate", json={"prompt": "7 8 9", **body})
            assert r.status_code == 200 and r.json()["token_ids"] == want_text["7 8 9"] and r.json()["finish_reason"] == "length"
            async with client.stream("POST", "/v1/generate", json={"prompt": "21 22", "modality": "image", "media": url, "stream": True,
                                                                  **body}) as resp:
                frames = [f for f in (await resp.aread()).decode().split("\n\n") if f]
            kinds = [f.split("\n")[0] for f in frames]
            assert kinds[0] == "event: accepted" and kinds[-1] == "event: done" and kinds.count("event: token") == 5
            assert json.loads(frames[-1].split("data: ", 1)[1])["token_ids"] == want_image
            answers = await asyncio.gather(*[client.post("/v1/generate", json={"prompt": p, **body}) for p in want_text])
            for p, a in zip(want_text, answers):
                assert a.status_code == 200 and a.json()["token_ids"] == want_text[p], p

    try:
        asyncio.run(scenario())
        assert rt.is_healthy
    finally:
        rt.stop()


@pytest.mark.parametrize("seed", range(6))
def test_repeated_restarts_at_random_steps_never_repeat_or_lose_a_token(seed):
    """Several engines in a row fail at random steps while requests of random lengths arrive at random times; every
    stream is exactly 101, 102, ... up to its length, once, whatever was in flight at each failure."""
    import random

    rnd = random.Random(seed)
    fail_steps = [rnd.randint(1, 12) for _ in range(4)]
    built = []

    def factory():
        built.append(FakeEngine(fail_after=fail_steps[len(built)] if len(built) < len(fail_steps) else None, step_delay=0.001))
        return built[-1]

    rt = ServingRuntime(factory, max_restarts=len(fail_steps))
    rt.start()
    try:
        lengths = [rnd.randint(1, 30) for _ in range(8)]
        handles = []
        for i, n in enumerate(lengths):
            handles.append(rt.submit(_req(f"r{i}", max_tokens=n)))
            time.sleep(rnd.choice([0.0, 0.002, 0.01]))
        for n, h in zip(lengths, handles):
            events = _drain(h, 30.0)
            assert [e.kind for e in events].count(EventKind.ACCEPTED) == 1
            assert [e.token_id for e in events if e.kind is EventKind.TOKEN] == list(range(101, 101 + n))
            assert events[-1].kind is EventKind.DONE and events[-1].token_ids == tuple(range(101, 101 + n))
        assert rt.is_healthy and len(rt.restarts) == len(built) - 1 <= len(fail_steps)
        assert rt.counters["accepted"] == 8 and rt.counters["finished"] == 8 and rt.counters["tokens"] == sum(lengths)
    finally:
        rt.stop()


def test_restart_allowance_counts_only_the_recent_window():
    """``max_restarts=1`` with a window: failures far apart are each survived, two inside one window are not."""
    plan = [2, 6, 6, 0]  # steps each engine in turn survives
    built = []

    def factory():
        built.append(FakeEngine(fail_after=plan[len(built)]))
        return built[-1]

    rt = ServingRuntime(factory, max_restarts=1, restart_window_s=0.2)
    rt.start()
    want = (101, 102, 103, 104)
    assert _drain(rt.submit(_req("a", max_tokens=4)))[-1].token_ids == want  # engine 1 fails at its step 3, engine 2 runs it again
    time.sleep(0.3)                                                           # the first restart leaves the window
    assert _drain(rt.submit(_req("b", max_tokens=4)))[-1].token_ids == want  # engine 2 fails at its step 7, engine 3 runs it again
    assert rt.is_healthy and len(built) == 3 and len(rt.restarts) == 2
    time.sleep(0.3)
    events = _drain(rt.submit(_req("c", max_tokens=50)))  # engine 3 fails at its step 7, engine 4 at once: two in one window
    assert events[-1].kind is EventKind.ERROR and "boom" in events[-1].error
    time.sleep(0.05)
    assert not rt.is_healthy and len(built) == 4 and len(rt.restarts) == 3
    rt.stop()


def test_a_rebuild_that_fails_ends_the_runtime():
    """The device no longer answers, say: the factory raises on the rebuild.  Open requests get the error and the
    runtime turns unhealthy, as without restarts."""
    built = []

    def factory():
        if built:
            raise RuntimeError("no device")
        built.append(FakeEngine(fail_after=2))
        return built[-1]

    rt = ServingRuntime(factory, max_restarts=3)
    rt.start()
    events = _drain(rt.submit(_req("z", max_tokens=50)))
    assert events[-1].kind is EventKind.ERROR and "no device" in events[-1].error
    time.sleep(0.05)
    assert not rt.is_healthy and "no device" in str(rt.failure) and len(rt.restarts) == 1 and built[0].exited
    with pytest.raises(RuntimeUnavailable):
        rt.submit(_req("late"))
    rt.stop()


def test_restart_with_the_real_engine_reproduces_the_stream():
    """The tiny engine on CPU fails once in the middle of decoding two requests (one with an image); after the rebuild
    both streams continue and equal the ones of an undisturbed engine, and /health names the restart."""
    import numpy as np
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights

    arch = Qwen3VLArch.tiny()
    weights = random_weights(arch, dtype=torch.float32, seed=0)
    image = Image.fromarray(np.random.default_rng(5).integers(0, 256, (64, 64, 3), dtype=np.uint8))
    built = []

    def make():
        eng = LLM("random:tiny", weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=64,
                  enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256, max_num_seqs=4)
        if not built:  # the first engine breaks on its fifth step
            inner, calls = eng.step_result, [0]

            def step_result():
                calls[0] += 1
                if calls[0] == 5:
                    raise RuntimeError("injected step failure")
                return inner()

            eng.step_result = step_result
        built.append(eng)
        return eng

    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    direct = LLM("random:tiny", weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=64,
                 enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256, max_num_seqs=4)
    want_text = direct.generate(["7 8 9"], sp)[0]["token_ids"]
    want_image = direct.generate_images("21 22", [image], sp)["token_ids"]
    direct.exit()

    rt = ServingRuntime(make, max_restarts=1)
    rt.start()
    try:
        h_text = rt.submit(GenerationRequest("t", "7 8 9", Modality.TEXT, None, sp))
        h_image = rt.submit(GenerationRequest("i", "21 22", Modality.IMAGE, image, sp))
        ev_text, ev_image = _drain(h_text, 60.0), _drain(h_image, 60.0)
        assert [e.token_id for e in ev_text if e.kind is EventKind.TOKEN] == want_text
        assert [e.token_id for e in ev_image if e.kind is EventKind.TOKEN] == want_image
        assert ev_text[-1].token_ids == tuple(want_text) and ev_image[-1].token_ids == tuple(want_image)
        assert len(built) == 2 and rt.restarts == ["RuntimeError: injected step failure"] and rt.is_healthy

        async def health():
            async with httpx.AsyncClient(transport=httpx.ASGITransport(app=create_app(rt, manage_runtime=False)), base_url="http://t") as c:
                return (await c.get("/health")).json()

        assert asyncio.run(health()) == {"status": "ok", "restarts": ["RuntimeError: injected step failure"]}
    finally:
        rt.stop()


def test_metrics_endpoint_reports_runtime_and_engine_numbers():
    """``/metrics`` (Prometheus text) and ``/v1/stats`` (JSON) of the tiny engine on CPU after a few requests: the
    runtime's own counters, scheduler counters, KV pages, prefix-cache counters and latency percentiles, published by
    the owner thread; every line of the text parses as ``name value`` with a TYPE line before it."""
    import numpy as np
    import torch
    from PIL import Image

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.models.architecture import Qwen3VLArch
    from prism_infer_b200.models.weights import random_weights
    from prism_infer_b200.serving.app import prometheus_text

    assert prometheus_text({"a-b": 1.0, "c": float("nan")}) == "# TYPE prism_a_b gauge\nprism_a_b 1.0\n# TYPE prism_c gauge\nprism_c NaN\n"
    weights = random_weights(Qwen3VLArch.tiny(), dtype=torch.float32, seed=0)
    rt = ServingRuntime(lambda: LLM("random:tiny", weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16,
                                    num_kvcache_blocks=64, enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256,
                                    max_num_seqs=4), stats_period_s=0.0)
    rt.start()
    try:
        sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
        image = Image.fromarray(np.random.default_rng(1).integers(0, 256, (64, 64, 3), dtype=np.uint8))
        for i in range(2):  # the second image request hits the multimodal prefix cache
            assert _drain(rt.submit(GenerationRequest(f"i{i}", f"{30 + i} 31", Modality.IMAGE, image, sp)), 60.0)[-1].kind is EventKind.DONE
        assert _drain(rt.submit(GenerationRequest("t", "7 8 9", Modality.TEXT, None, sp)), 60.0)[-1].kind is EventKind.DONE
        h = rt.submit(GenerationRequest("c", "7 8 9", Modality.TEXT, None, SamplingParams(temperature=0.0, max_tokens=200, ignore_eos=True)))
        assert h.next_event_blocking(30.0).kind is EventKind.ACCEPTED
        rt.cancel("c")
        assert _drain(h, 60.0)[-1].finish_reason == "cancelled"
        time.sleep(0.05)  # one more pass of the owner thread publishes the final numbers

        async def scrape():
            async with httpx.AsyncClient(transport=httpx.ASGITransport(app=create_app(rt, manage_runtime=False)), base_url="http://t") as c:
                return (await c.get("/metrics")), (await c.get("/v1/stats"))

        text, js = asyncio.run(scrape())
        assert text.status_code == 200 and text.headers["content-type"].startswith("text/plain")
        lines = text.text.strip().split("\n")
        parsed = {}
        for type_line, value_line in zip(lines[0::2], lines[1::2]):
            name, value = value_line.split(" ")
            assert type_line == f"# TYPE {name} gauge" and name.startswith("prism_")
            parsed[name[len("prism_"):]] = float(value)
        stats = js.json()
        assert parsed.keys() == stats.keys()
        assert stats["healthy"] == 1.0 and stats["restarts"] == 0.0 and stats["runtime_open_requests"] == 0.0
        assert stats["runtime_accepted"] == 4.0 and stats["runtime_finished"] == 3.0 and stats["runtime_cancelled"] == 1.0
        assert stats["runtime_tokens"] >= 12.0 and stats["runtime_steps"] >= 6.0
        assert stats["engine_scheduler_admitted"] == 4.0 and stats["engine_scheduler_finished"] == 3.0 and stats["engine_scheduler_cancelled"] == 1.0
        assert stats["engine_kv_pages_total"] == 64.0 and 0.0 < stats["engine_kv_pages_used"] < 64.0  # the cached image prefix stays resident
        assert stats["engine_prefix_cache_hits"] == 1.0 and stats["engine_prefix_cache_entries"] >= 1.0
        assert stats["engine_latency_window_requests"] == 4.0
        assert 0.0 < stats["engine_ttft_ms_p50"] <= stats["engine_ttft_ms_p99"] and stats["engine_tpot_ms_p50"] > 0.0
    finally:
        rt.stop()


def test_prism_serve_process_answers_over_tcp(tmp_path):
    """The console entry as a user starts it: a child process (``python -m prism_infer_b200.serving.cli``) with an engine
    configuration file, the tiny model on CPU, a real socket; health, one generation, then a clean shutdown on SIGTERM."""
    import os
    import signal
    import socket
    import subprocess
    import sys
    import time
    import urllib.request

    cfg = tmp_path / "engine.json"
    cfg.write_text(json.dumps({"device": "cpu", "max_model_len": 128, "kvcache_block_size": 16, "num_kvcache_blocks": 16, "enforce_eager": True}))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.Popen([sys.executable, "-m", "prism_infer_b200.serving.cli", "--model", "random:tiny", "--engine-config", str(cfg),
                             "--host", "127.0.0.1", "--port", str(port), "--log-level", "warning"], cwd=root,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    try:
        deadline = time.time() + 90
        while True:
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                pass
            assert proc.poll() is None, proc.stdout.read().decode()[-2000:]
            assert time.time() < deadline, "the server did not come up"
            time.sleep(0.3)
        body = json.dumps({"prompt": "7 8 9", "sampling": {"max_tokens": 4, "ignore_eos": True}}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/generate", data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            out = json.loads(r.read())
        assert out["event"] == "done" and len(out["token_ids"]) == 4 and out["finish_reason"] == "length"
        # the same server through its other doors: the chat protocol, the model list, the metrics
        body = json.dumps({"messages": [{"role": "user", "content": "7 8 9"}], "max_tokens": 4}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body, headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=60) as r:
            chat = json.loads(r.read())
        assert chat["object"] == "chat.completion" and chat["choices"][0]["message"]["role"] == "assistant"
        assert 1 <= chat["usage"]["completion_tokens"] <= 4 and chat["choices"][0]["finish_reason"] in ("stop", "length")
        assert chat["usage"]["prompt_tokens"] == out["prompt_tokens"] >= 3  # the same prompt through both doors
        assert chat["usage"]["total_tokens"] == chat["usage"]["prompt_tokens"] + chat["usage"]["completion_tokens"]
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/v1/models", timeout=10) as r:
            assert json.loads(r.read())["data"][0]["id"] == "random:tiny"
        time.sleep(1.2)  # the owner thread publishes its numbers once a second
        with urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10) as r:
            text = r.read().decode()
        assert "prism_runtime_accepted 2.0" in text and "prism_healthy 1.0" in text and "prism_engine_kv_pages_total 16.0" in text
    finally:
        proc.send_signal(signal.SIGTERM)  # this exact child; uvicorn turns the signal into a lifespan shutdown
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait(timeout=10)
    assert proc.returncode in (0, -signal.SIGTERM), proc.returncode
