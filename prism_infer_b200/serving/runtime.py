"""Serving runtime: one owner thread builds and drives the engine.

Everything that touches the engine (construction, admission, stepping, cancellation,
shutdown) happens on a single "engine owner" thread; the ASGI event loop only talks to it
through a bounded ingress queue and per-request event queues filled with
``loop.call_soon_threadsafe``.  Behaviour follows ``prism_infer/serving/runtime.py:143-583``:
a full ingress queue raises ``IngressFull`` (HTTP 429), a duplicate id ``DuplicateRequest``
(409), every emitted token becomes a ``TOKEN`` event with its single-token text, ``DONE``
carries the full text, shutdown cancels everything with ``finish_reason="shutdown"``, and an
engine failure sends ``ERROR`` to every open request and flips ``is_healthy``.
"""

from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Protocol

from ..engine.contracts import StepResult
from .protocol import EventKind, GenerationRequest, Modality, ServingEvent


class ServingEngine(Protocol):
    """What the runtime needs from an engine (``LLM`` satisfies it)."""

    tokenizer: Any

    def add_request(self, prompt, sampling_params=None, *, raise_on_reject: bool = True) -> int: ...
    def add_vl_request(self, prompt, image, sampling_params=None, **kw) -> int: ...
    def add_images_request(self, prompt, images, sampling_params=None, **kw) -> int: ...
    def add_video_request(self, prompt, frames, sampling_params=None, **kw) -> int: ...
    def step_result(self) -> StepResult: ...
    def is_finished(self) -> bool: ...
    def cancel_request(self, request_id: int) -> bool: ...
    def request_state(self, request_id: int): ...
    def exit(self) -> None: ...


class IngressFull(RuntimeError):
    pass


class DuplicateRequest(RuntimeError):
    pass


class RuntimeUnavailable(RuntimeError):
    pass


class RequestHandle:
    """Consumer side of one request's event stream (lives on the asyncio loop)."""

    def __init__(self, request_id: str, loop: asyncio.AbstractEventLoop | None) -> None:
        self.request_id = request_id
        self._loop = loop
        self._queue: "asyncio.Queue[ServingEvent] | queue.Queue[ServingEvent]" = (
            asyncio.Queue() if loop is not None else queue.Queue())
        self.closed = False

    def publish(self, event: ServingEvent) -> None:
        """Called from the engine thread."""
        if self._loop is not None:
            self._loop.call_soon_threadsafe(self._queue.put_nowait, event)
        else:
            self._queue.put_nowait(event)

    async def next_event(self) -> ServingEvent:
        return await self._queue.get()  # type: ignore[misc]

    def next_event_blocking(self, timeout: float | None = None) -> ServingEvent:
        return self._queue.get(timeout=timeout)  # type: ignore[call-arg]


@dataclass
class _Live:
    request: GenerationRequest
    handle: RequestHandle
    engine_id: int | None = None
    token_ids: list[int] = field(default_factory=list)
    prompt_tokens: int | None = None
    replayed: int = 0  # after an engine restart: how many of the tokens already delivered the new engine has produced again


class ServingRuntime:
    """``max_restarts`` (default 0: a failure of the engine ends the runtime, as in the reference): after a failure in a step
    the engine is closed, a new one is built by the factory and every open greedy request is submitted again; the tokens
    it had already delivered are produced a second time, checked against what was delivered and not sent twice.  Requests
    that sample (temperature > 0) cannot be reproduced and end with an error.  A fault that leaves the device unusable
    also fails the rebuild, which ends the runtime."""

    def __init__(self, engine_factory: Callable[[], ServingEngine], *, ingress_capacity: int = 64,
                 idle_sleep_s: float = 0.001, max_restarts: int = 0, restart_window_s: float = 0.0,
                 stats_period_s: float = 1.0) -> None:
        self._factory = engine_factory
        self.max_restarts = int(max_restarts)
        # 0: the allowance is for the runtime's whole life; otherwise only restarts of the last ``restart_window_s``
        # seconds count, so a server that runs for weeks survives rare faults but still gives up on a fault that repeats
        self.restart_window_s = float(restart_window_s)
        self._restart_times: list[float] = []
        self.restarts: list[str] = []  # one line per restart: the failure that caused it
        self._ingress: "queue.Queue[_Live]" = queue.Queue(maxsize=ingress_capacity)
        self._cancel: "queue.Queue[str]" = queue.Queue()
        self._cancel_early: set[str] = set()  # owner thread only
        self._live: dict[str, _Live] = {}
        self._by_engine: dict[int, _Live] = {}
        self._ids: set[str] = set()
        self._ids_lock = threading.Lock()
        self._thread: threading.Thread | None = None
        self._ready = threading.Event()
        self._stop = threading.Event()
        self._idle_sleep_s = idle_sleep_s
        self.engine: ServingEngine | None = None
        self.failure: BaseException | None = None
        self.steps = 0
        self.counters = {"accepted": 0, "finished": 0, "errors": 0, "cancelled": 0, "tokens": 0}
        self._stats_period_s = float(stats_period_s)
        self._stats_due = 0.0
        self._stats: dict[str, float] = {}

    # ------------------------------------------------------------------ lifecycle
    @property
    def is_healthy(self) -> bool:
        return self._thread is not None and self._thread.is_alive() and self.failure is None and self._ready.is_set()

    def start(self, timeout_s: float = 600.0) -> None:
        if self._thread is not None:
            raise RuntimeError("runtime already started")
        self._thread = threading.Thread(target=self._run, name="prism-engine-owner", daemon=True)
        self._thread.start()
        if not self._ready.wait(timeout_s):
            raise RuntimeUnavailable("engine did not start in time")
        if self.failure is not None:
            raise RuntimeUnavailable(f"engine failed to start: {self.failure}")

    def stop(self, timeout_s: float = 30.0) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout_s)

    def stats(self) -> dict[str, float]:
        """Flat ``name -> number``: the runtime's own counters plus the engine's ``serving_stats()`` as the owner thread
        last published them (every ``stats_period_s`` between steps; the HTTP side never reads the engine itself)."""
        return {**self._stats, "healthy": float(self.is_healthy), "ingress_depth": float(self._ingress.qsize()),
                "restarts": float(len(self.restarts))}

    def _publish_stats(self, force: bool = False) -> None:
        now = time.monotonic()
        if not force and now < self._stats_due:
            return
        self._stats_due = now + self._stats_period_s
        stats = {f"runtime_{k}": float(v) for k, v in self.counters.items()}
        stats["runtime_steps"] = float(self.steps)
        stats["runtime_open_requests"] = float(len(self._live))
        probe = getattr(self.engine, "serving_stats", None)
        if probe is not None:
            try:
                stats.update({f"engine_{k}": float(v) for k, v in probe().items()})
            except Exception:  # a summary must never take the engine thread down
                stats["runtime_stats_failures"] = self._stats.get("runtime_stats_failures", 0.0) + 1.0
        self._stats = stats  # one reference assignment: readers see the old or the new dictionary, never a mix

    # --------------------------------------------------------------------- ingress
    def submit(self, request: GenerationRequest, loop: asyncio.AbstractEventLoop | None = None) -> RequestHandle:
        if not self.is_healthy:
            raise RuntimeUnavailable(f"engine is not available: {self.failure}" if self.failure else "engine is not running")
        with self._ids_lock:
            if request.request_id in self._ids:
                raise DuplicateRequest(f"request id {request.request_id!r} is already in flight")
            self._ids.add(request.request_id)
        handle = RequestHandle(request.request_id, loop)
        try:
            self._ingress.put_nowait(_Live(request, handle))
        except queue.Full:
            with self._ids_lock:
                self._ids.discard(request.request_id)
            raise IngressFull(f"ingress queue is full ({self._ingress.maxsize} requests)") from None
        return handle

    def cancel(self, request_id: str) -> None:
        self._cancel.put(request_id)

    def is_open(self, request_id: str) -> bool:
        """Submitted and not finished yet (queued for admission or running)."""
        with self._ids_lock:
            return request_id in self._ids

    # ---------------------------------------------------------------- engine thread
    def _finish(self, live: _Live, event: ServingEvent) -> None:
        self.counters["errors" if event.kind is EventKind.ERROR else
                      "cancelled" if event.finish_reason == "cancelled" else "finished"] += 1
        # the books are closed before the final event goes out: a client that sees it may reuse the id at once
        self._live.pop(live.request.request_id, None)
        if live.engine_id is not None:
            self._by_engine.pop(live.engine_id, None)
        with self._ids_lock:
            self._ids.discard(live.request.request_id)
        live.handle.publish(event)
        live.handle.closed = True

    def _admit(self, live: _Live, *, replay: bool = False) -> None:
        eng, req = self.engine, live.request
        assert eng is not None
        if req.request_id in self._cancel_early:  # cancelled while it waited for admission: never reaches the engine
            self._cancel_early.discard(req.request_id)
            self._finish(live, ServingEvent(req.request_id, EventKind.DONE, text="", finish_reason="cancelled"))
            return
        try:
            if req.modality is Modality.TEXT:
                eid = eng.add_request(req.prompt, req.sampling_params, raise_on_reject=False)
            elif req.modality is Modality.IMAGE:
                media = req.media
                if isinstance(media, tuple):
                    eid = eng.add_images_request(req.prompt, list(media), req.sampling_params, raise_on_reject=False)
                else:
                    eid = eng.add_vl_request(req.prompt, media, req.sampling_params, raise_on_reject=False)
            else:
                frames = list(req.media) if isinstance(req.media, (tuple, list)) else req.media
                eid = eng.add_video_request(req.prompt, frames, req.sampling_params, raise_on_reject=False)
        except Exception as exc:  # invalid media, tokenizer failure, ...
            self._finish(live, ServingEvent(req.request_id, EventKind.ERROR, error=f"{type(exc).__name__}: {exc}"))
            return
        live.engine_id = eid
        if req.ttft_slo_ms is not None and hasattr(eng, "set_first_token_deadline"):
            eng.set_first_token_deadline(eid, req.ttft_slo_ms)
        count = getattr(eng, "prompt_token_count", None)
        live.prompt_tokens = count(eid) if count is not None else None
        self._live[req.request_id] = live
        self._by_engine[eid] = live
        if not replay:
            self.counters["accepted"] += 1
            live.handle.publish(ServingEvent(req.request_id, EventKind.ACCEPTED, engine_request_id=eid))
        state = eng.request_state(eid)
        if state is not None and getattr(state, "value", "") == "rejected":
            self._finish(live, ServingEvent(req.request_id, EventKind.DONE, engine_request_id=eid, text="",
                                            finish_reason="rejected"))

    def _apply_cancellations(self) -> None:
        while True:
            try:
                rid = self._cancel.get_nowait()
            except queue.Empty:
                return
            live = self._live.get(rid)
            if live is None or live.engine_id is None:
                if self.is_open(rid):
                    self._cancel_early.add(rid)  # still in the ingress queue: cancelled when it is taken out
                continue
            self.engine.cancel_request(live.engine_id)  # type: ignore[union-attr]
            self._finish(live, self._done(live, "cancelled"))

    def _done(self, live: _Live, reason: str) -> ServingEvent:
        text = self.engine.tokenizer.decode(live.token_ids) if live.token_ids else ""  # type: ignore[union-attr]
        return ServingEvent(live.request.request_id, EventKind.DONE, engine_request_id=live.engine_id,
                            token_ids=tuple(live.token_ids), text=text, finish_reason=reason, prompt_tokens=live.prompt_tokens)

    def _drain_ingress(self) -> None:
        while True:
            try:
                live = self._ingress.get_nowait()
            except queue.Empty:
                return
            self._admit(live)

    def _restart(self, cause: BaseException) -> None:
        """Close the failed engine, build a new one and submit the open requests again (see the class docstring)."""
        self.restarts.append(f"{type(cause).__name__}: {cause}")
        try:
            self.engine.exit()  # type: ignore[union-attr]
        except Exception:
            pass
        self.engine = self._factory()
        open_requests = list(self._live.values())
        self._live.clear()
        self._by_engine.clear()
        for live in open_requests:
            live.engine_id, live.replayed = None, 0  # ids of the old engine mean nothing to the new one
            if live.request.sampling_params.temperature > 0:
                self._finish(live, ServingEvent(live.request.request_id, EventKind.ERROR,
                                                error="the engine was restarted and a sampled request cannot be reproduced"))
                continue
            self._admit(live, replay=True)

    def _deliver(self, live: _Live, out) -> None:
        if out.new_token is not None:
            if live.replayed < len(live.token_ids):
                # a token the client already has: it must come out the same, and is not sent again
                if live.token_ids[live.replayed] != out.new_token:
                    self.engine.cancel_request(out.request_id)  # type: ignore[union-attr]
                    self._finish(live, ServingEvent(live.request.request_id, EventKind.ERROR,
                                                    error="the restarted engine did not reproduce the tokens already delivered"))
                    return
                live.replayed += 1
            else:
                live.token_ids.append(out.new_token)
                live.replayed = len(live.token_ids)
                self.counters["tokens"] += 1
                live.handle.publish(ServingEvent(
                    live.request.request_id, EventKind.TOKEN, engine_request_id=out.request_id,
                    token_id=out.new_token, token_text=self.engine.tokenizer.decode([out.new_token])))  # type: ignore[union-attr]
        if out.finished:
            self._finish(live, self._done(live, out.finish_reason or "finished"))

    def _run(self) -> None:
        try:
            self.engine = self._factory()
        except BaseException as exc:  # noqa: BLE001
            self.failure = exc
            self._ready.set()
            return
        self._ready.set()
        try:
            while not self._stop.is_set():
                try:
                    self._apply_cancellations()
                    self._drain_ingress()
                    self._publish_stats()
                    if self.engine.is_finished():
                        time.sleep(self._idle_sleep_s)
                        continue
                    result = self.engine.step_result()
                except Exception as exc:  # a failed step: rebuild and replay while restarts are left
                    now = time.monotonic()
                    recent = [t for t in self._restart_times if self.restart_window_s <= 0 or now - t < self.restart_window_s]
                    if len(recent) >= self.max_restarts or self._stop.is_set():
                        raise
                    self._restart_times = recent + [now]
                    self._restart(exc)
                    continue
                self.steps += 1
                for out in result.outputs:
                    live = self._by_engine.get(out.request_id)
                    if live is not None:
                        self._deliver(live, out)
        except BaseException as exc:  # noqa: BLE001 - reported to every open request
            self.failure = exc
            for live in list(self._live.values()):
                self._finish(live, ServingEvent(live.request.request_id, EventKind.ERROR,
                                                error=f"engine failure: {type(exc).__name__}: {exc}"))
        finally:
            for live in list(self._live.values()):
                if live.engine_id is not None:
                    try:
                        self.engine.cancel_request(live.engine_id)
                    except Exception:
                        pass
                self._finish(live, self._done(live, "shutdown"))
            while True:  # requests that never reached the engine
                try:
                    live = self._ingress.get_nowait()
                except queue.Empty:
                    break
                self._finish(live, ServingEvent(live.request.request_id, EventKind.DONE, text="", finish_reason="shutdown"))
            try:
                self.engine.exit()
            except Exception:
                pass
