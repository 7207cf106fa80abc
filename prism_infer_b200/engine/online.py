"""Deterministic open-loop arrival driver and the media preprocessing caches (reference
``prism_infer/engine/online.py:240-955``).

``OnlineServingSession.run`` replays a list of ``OnlineRequest``s: each becomes visible at
its arrival offset, media preprocessing runs on a one-worker background pool, admission
and stepping stay on the calling (engine) thread, cancellations fire at their offsets, and
per-request TTFT / end-to-end latency are measured from the *planned* arrival time, so
queueing and preprocessing count.  Clock and sleep are injectable (tests use a fake clock).

Caches (all content-addressed, nothing keyed by object identity):

* processor-output cache: SHA-256 over the media bytes -> patches + grids (LRU, 128 entries);
* layout cache with prompt rebinding: a media set seen before keeps its placeholder prefix;
  a new question about it is only tokenised and spliced behind that prefix;
* the fingerprint doubles as ``multimodal_prefix_cache_key`` / ``visual_embedding_cache_key``.
"""

from __future__ import annotations

import hashlib
import time
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from math import isfinite
from typing import Any, Callable, Iterable, Sequence as Seq

import numpy as np
import torch

from ..sampling_params import SamplingParams
from .vl_inputs import ImageInputs, VideoInputs, image_block, to_uint8_hwc, video_blocks

PAYLOAD_TYPES = ("text", "image", "images", "interleaved_images", "video")


def media_fingerprint(*items: Any) -> str:
    """SHA-256 over the content of bytes / PIL / numpy / torch / path / str items."""
    h = hashlib.sha256()
    for it in items:
        if isinstance(it, (bytes, bytearray)):
            h.update(b"b")
            h.update(bytes(it))
        elif isinstance(it, torch.Tensor):
            a = it.detach().cpu().contiguous()
            h.update(f"t{tuple(a.shape)}{a.dtype}".encode())
            h.update(a.view(torch.uint8).numpy().tobytes())
        elif isinstance(it, np.ndarray):
            a = np.ascontiguousarray(it)
            h.update(f"n{a.shape}{a.dtype}".encode())
            h.update(a.tobytes())
        elif isinstance(it, str):
            h.update(b"s" + it.encode("utf-8"))
        elif isinstance(it, (list, tuple)):
            h.update(f"l{len(it)}".encode())
            h.update(media_fingerprint(*it).encode())
        elif hasattr(it, "tobytes") and hasattr(it, "size"):  # PIL image
            h.update(f"p{it.size}{getattr(it, 'mode', '')}".encode())
            h.update(it.tobytes())
        else:
            h.update(repr(it).encode())
    return h.hexdigest()


@dataclass(frozen=True)
class OnlineRequest:
    request_key: str
    arrival_offset_s: float
    payload: dict[str, Any]
    sampling_params: SamplingParams
    cancel_offset_s: float | None = None
    ttft_slo_ms: float | None = None

    def __post_init__(self) -> None:
        if not isinstance(self.request_key, str) or not self.request_key:
            raise ValueError("request_key must not be empty")
        if not isfinite(float(self.arrival_offset_s)) or self.arrival_offset_s < 0:
            raise ValueError("arrival_offset_s must be a finite non-negative number")
        kind = self.payload.get("type")
        if kind not in PAYLOAD_TYPES:
            raise ValueError(f"payload type must be one of {PAYLOAD_TYPES}, got {kind!r}")
        if "prompt" not in self.payload:
            raise ValueError("payload needs a prompt")
        if not isinstance(self.sampling_params, SamplingParams):
            raise TypeError("online request sampling_params must be SamplingParams")
        if self.cancel_offset_s is not None and self.cancel_offset_s < self.arrival_offset_s:
            raise ValueError("cancel_offset_s must not precede the arrival")
        if self.ttft_slo_ms is not None and (not isfinite(float(self.ttft_slo_ms)) or self.ttft_slo_ms <= 0):
            raise ValueError("ttft_slo_ms must be a finite positive number or None")


@dataclass
class OnlineRequestResult:
    request_key: str
    engine_request_id: int | None
    arrival_offset_s: float
    token_ids: list[int] = field(default_factory=list)
    finish_reason: str | None = None
    ttft_ms: float | None = None
    latency_ms: float | None = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    preprocess_ms: float = 0.0

    def to_record(self) -> dict[str, object]:
        return dict(self.__dict__)


@dataclass
class OnlineRunResult:
    requests: list[OnlineRequestResult]
    started_ns: int
    finished_ns: int
    steps: int
    cache_counters: dict[str, int]

    @property
    def duration_s(self) -> float:
        return (self.finished_ns - self.started_ns) / 1e9

    def to_record(self) -> dict[str, object]:
        return {"duration_s": self.duration_s, "steps": self.steps, "cache_counters": dict(self.cache_counters),
                "requests": [r.to_record() for r in self.requests]}


class _LRU(OrderedDict):
    def __init__(self, capacity: int) -> None:
        super().__init__()
        self.capacity = capacity

    def get_refresh(self, key):
        if key in self:
            self.move_to_end(key)
            return self[key]
        return None

    def put(self, key, value) -> None:
        self[key] = value
        self.move_to_end(key)
        while len(self) > self.capacity:
            self.popitem(last=False)


class OnlineServingSession:
    def __init__(self, engine, *, clock_ns: Callable[[], int] = time.perf_counter_ns,
                 sleep: Callable[[float], None] = time.sleep, processor_cache_entries: int = 128,
                 background_preprocessing: bool = True) -> None:
        self.engine = engine
        self.clock_ns = clock_ns
        self.sleep = sleep
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="prism-preprocess") if background_preprocessing else None
        self._patch_cache = _LRU(processor_cache_entries)     # fingerprint of one item -> (patches, grid)
        self._layout_cache = _LRU(processor_cache_entries)    # fingerprint of the media set -> prefix ids + tensors
        self._fingerprints: dict[int, str] = {}                # id(obj) memo, valid only within one run
        self.counters = {"processor_hits": 0, "processor_misses": 0, "layout_hits": 0, "layout_misses": 0,
                         "rebinds": 0, "fingerprint_memo_hits": 0}

    # ------------------------------------------------------------------ preprocessing
    def _fingerprint(self, obj: Any) -> str:
        memo = self._fingerprints.get(id(obj))
        if memo is not None:
            self.counters["fingerprint_memo_hits"] += 1
            return memo
        if hasattr(obj, "convert") or isinstance(obj, (np.ndarray, torch.Tensor)):
            fp = media_fingerprint(to_uint8_hwc(obj))
        else:
            fp = media_fingerprint(obj)
        self._fingerprints[id(obj)] = fp
        return fp

    def _patches(self, item: Any, *, video_frames: Seq[Any] | None = None):
        proc = self.engine.processor
        if video_frames is not None:
            key = "v:" + media_fingerprint(*[self._fingerprint(f) for f in video_frames])
        else:
            key = "i:" + self._fingerprint(item)
        hit = self._patch_cache.get_refresh(key)
        if hit is not None:
            self.counters["processor_hits"] += 1
            return key, hit
        self.counters["processor_misses"] += 1
        out = proc.process_video(list(video_frames)) if video_frames is not None else proc.process_image(item)
        self._patch_cache.put(key, out)
        return key, out

    def _stage(self, pixels: torch.Tensor) -> torch.Tensor:
        """Patches of a cached layout in the form the runner copies from (pinned bf16 on CUDA
        engines): converted once here, off the submission path, and reused by every later hit."""
        stage = getattr(self.engine, "stage_pixels", None)
        return stage(pixels) if stage is not None else pixels

    def prepare_media(self, payload: dict[str, Any]) -> tuple[ImageInputs | VideoInputs, str]:
        """Processor output for a media payload plus its content key, through the caches."""
        arch, tok = self.engine.arch, self.engine.tokenizer
        kind = payload["type"]
        prompt = payload["prompt"]
        if kind == "video":
            frames = payload.get("frames", payload.get("video"))
            key, (pv, grid) = self._patches(None, video_frames=frames)
            layout = self._layout_cache.get_refresh(key)
            if layout is None:
                self.counters["layout_misses"] += 1
                layout = (video_blocks(arch, grid, arch.vision.merge_unit), self._stage(pv), [grid])
                self._layout_cache.put(key, layout)
            else:
                self.counters["layout_hits"] += 1
                self.counters["rebinds"] += 1
            prefix, pv, grids = layout
            ids = list(prefix) + (tok.encode(prompt) if isinstance(prompt, str) else list(prompt))
            return VideoInputs(ids, pv, list(grids)), key
        images = [payload["image"]] if kind == "image" else list(payload["images"])
        parts = [self._patches(img) for img in images]
        key = "m:" + media_fingerprint(*[k for k, _ in parts])
        if kind == "interleaved_images":
            marker = payload.get("image_marker", "<image>")
            segments = prompt.split(marker)
            if len(segments) - 1 != len(images):
                raise ValueError(f"prompt has {len(segments) - 1} {marker!r} markers for {len(images)} images")
            last = segments[-1]
            lkey = key + ":" + hashlib.sha256(marker.join(segments[:-1]).encode()).hexdigest()
            layout = self._layout_cache.get_refresh(lkey)
            if layout is None:
                self.counters["layout_misses"] += 1
                ids: list[int] = []
                for i, (_, (pv, grid)) in enumerate(parts):
                    if segments[i].strip():
                        ids += tok.encode(segments[i])
                    ids += image_block(arch, self.engine.processor.tokens_for(grid))
                layout = (ids, self._stage(torch.cat([pv for _, (pv, _) in parts])), [g for _, (_, g) in parts])
                self._layout_cache.put(lkey, layout)
            else:
                self.counters["layout_hits"] += 1
                self.counters["rebinds"] += 1
            prefix, pv, grids = layout
            ids = list(prefix) + (tok.encode(last) if last.strip() else [])
            return ImageInputs(ids, pv, list(grids)), key
        layout = self._layout_cache.get_refresh(key)
        if layout is None:
            self.counters["layout_misses"] += 1
            ids = []
            for _, (pv, grid) in parts:
                ids += image_block(arch, self.engine.processor.tokens_for(grid))
            layout = (ids, self._stage(torch.cat([pv for _, (pv, _) in parts])), [g for _, (_, g) in parts])
            self._layout_cache.put(key, layout)
        else:
            self.counters["layout_hits"] += 1
            self.counters["rebinds"] += 1
        prefix, pv, grids = layout
        ids = list(prefix) + (tok.encode(prompt) if isinstance(prompt, str) else list(prompt))
        return ImageInputs(ids, pv, list(grids)), key

    # ------------------------------------------------------------------------ run
    def _admit(self, req: OnlineRequest, prepared, arrival_ns: int) -> int:
        eng = self.engine
        kind = req.payload["type"]
        if kind == "text":
            seq_kwargs = dict(raise_on_reject=False)
            rid = eng.add_request(req.payload["prompt"], req.sampling_params, **seq_kwargs)
            if req.ttft_slo_ms is not None:
                eng.set_first_token_deadline(rid, req.ttft_slo_ms)  # counted from the engine's own arrival stamp
        else:
            inputs, key = prepared
            seq = eng._multimodal_sequence(inputs, req.sampling_params, media_key=key)
            seq.arrival_ns = arrival_ns
            if req.ttft_slo_ms is not None:
                seq.deadline_ns = arrival_ns + int(req.ttft_slo_ms * 1e6)
            rid = eng._submit(seq, raise_on_reject=False)
        return rid

    def run(self, requests: Iterable[OnlineRequest]) -> OnlineRunResult:
        reqs = sorted(requests, key=lambda r: r.arrival_offset_s)
        keys = [r.request_key for r in reqs]
        if len(set(keys)) != len(keys):
            raise ValueError("request keys must be unique")
        eng = self.engine
        self._fingerprints.clear()
        t0 = self.clock_ns()
        results = {r.request_key: OnlineRequestResult(r.request_key, None, r.arrival_offset_s) for r in reqs}
        pending_prep: list[tuple[OnlineRequest, Future | None, Any, int]] = []
        by_engine: dict[int, OnlineRequest] = {}
        cancels = sorted((r for r in reqs if r.cancel_offset_s is not None), key=lambda r: r.cancel_offset_s)
        next_arrival = 0
        steps = 0
        open_keys: set[str] = set()

        def now_s() -> float:
            return (self.clock_ns() - t0) / 1e9

        while True:
            t = now_s()
            while next_arrival < len(reqs) and reqs[next_arrival].arrival_offset_s <= t:
                r = reqs[next_arrival]
                next_arrival += 1
                arrival_ns = t0 + int(r.arrival_offset_s * 1e9)
                if r.payload["type"] == "text":
                    pending_prep.append((r, None, None, arrival_ns))
                elif self._pool is not None:
                    pending_prep.append((r, self._pool.submit(self._timed_prepare, r.payload), None, arrival_ns))
                else:
                    pending_prep.append((r, None, self._timed_prepare(r.payload), arrival_ns))
            still: list = []
            for r, fut, ready, arrival_ns in pending_prep:
                if fut is not None and not fut.done():
                    still.append((r, fut, ready, arrival_ns))
                    continue
                prepared, prep_ms = (None, 0.0)
                if r.payload["type"] != "text":
                    try:
                        prepared, prep_ms = fut.result() if fut is not None else ready
                    except Exception as exc:
                        results[r.request_key].finish_reason = f"preprocess_error: {type(exc).__name__}: {exc}"
                        continue
                rid = self._admit(r, prepared, arrival_ns)
                res = results[r.request_key]
                res.engine_request_id, res.preprocess_ms = rid, prep_ms
                seq = eng._sequences.get(rid)
                if seq is None:
                    res.finish_reason = "rejected"
                    continue
                seq.arrival_ns = arrival_ns
                metric = eng.metrics.requests.get(rid)
                if metric is not None:
                    metric.submitted_ns = arrival_ns
                res.prompt_tokens = seq.num_prompt_tokens
                by_engine[rid] = r
                open_keys.add(r.request_key)
            pending_prep = still
            while cancels and cancels[0].cancel_offset_s <= t:
                c = cancels.pop(0)
                res = results[c.request_key]
                if c.request_key in open_keys and res.engine_request_id is not None:
                    eng.cancel_request(res.engine_request_id)
                    res.finish_reason = "cancelled"
                    res.latency_ms = (self.clock_ns() - (t0 + int(c.arrival_offset_s * 1e9))) / 1e6
                    open_keys.discard(c.request_key)
            if not eng.is_finished():
                step = eng.step_result()
                steps += 1
                now = self.clock_ns()
                for out in step.outputs:
                    r = by_engine.get(out.request_id)
                    if r is None or r.request_key not in open_keys:
                        continue
                    res = results[r.request_key]
                    arrival_ns = t0 + int(r.arrival_offset_s * 1e9)
                    if out.new_token is not None:
                        if not res.token_ids:
                            res.ttft_ms = (now - arrival_ns) / 1e6
                        res.token_ids.append(out.new_token)
                    if out.finished:
                        res.finish_reason = out.finish_reason
                        res.latency_ms = (now - arrival_ns) / 1e6
                        m = eng.metrics.requests.get(out.request_id)
                        if m is not None:
                            res.cached_tokens = m.cached_tokens
                        open_keys.discard(r.request_key)
                continue
            if next_arrival >= len(reqs) and not pending_prep and not open_keys:
                break
            # idle: wait for the next arrival, cancellation or preprocessing result
            waits = []
            if next_arrival < len(reqs):
                waits.append(reqs[next_arrival].arrival_offset_s - now_s())
            if cancels:
                waits.append(cancels[0].cancel_offset_s - now_s())
            delay = min(waits) if waits else 0.0005
            self.sleep(max(0.0, min(delay, 0.001) if pending_prep else max(0.0, delay)))
        return OnlineRunResult([results[k] for k in keys], t0, self.clock_ns(), steps, dict(self.counters))

    def _timed_prepare(self, payload: dict[str, Any]):
        t = time.perf_counter()
        out = self.prepare_media(payload)
        return out, (time.perf_counter() - t) * 1e3

    def reset_metrics(self) -> None:
        self.engine.reset_metrics()
        for k in self.counters:
            self.counters[k] = 0

    def close(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
