"""FastAPI application: ``GET /health``, ``POST /v1/generate`` (JSON or SSE) and, beyond the reference, ``GET /metrics``
(Prometheus text), ``GET /v1/stats`` (the same numbers as JSON) and the OpenAI-style ``POST /v1/chat/completions`` /
``GET /v1/models`` of ``openai_api.py``.

Same wire contract as the reference (``prism_infer/serving/app.py:36-267``): strict
pydantic bodies (unknown fields rejected), media as ``data:image/...;base64`` URLs or path
strings, video as an explicit list of frame data-URLs, SSE frames
``event: <kind>\\ndata: <json>\\n\\n``, client disconnect cancels the request, and status
codes 400 (bad request / engine-side error), 409 (duplicate id), 429 (ingress full),
499 (client went away), 503 (engine down).
"""

from __future__ import annotations

import asyncio
import base64
import io
import json
import uuid
from contextlib import asynccontextmanager
from typing import Annotated, AsyncIterator, Literal

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse
from pydantic import BaseModel, ConfigDict, Field, model_validator

from ..sampling_params import SamplingParams
from .protocol import EventKind, GenerationRequest, Modality, ServingEvent
from .runtime import DuplicateRequest, IngressFull, RequestHandle, RuntimeUnavailable, ServingRuntime


class SamplingBody(BaseModel):
    model_config = ConfigDict(extra="forbid")
    temperature: Annotated[float, Field(ge=0.0)] = 0.0
    max_tokens: Annotated[int, Field(gt=0)] = 64
    ignore_eos: bool = False


class GenerateBody(BaseModel):
    model_config = ConfigDict(extra="forbid")
    request_id: str | None = None
    prompt: Annotated[str, Field(min_length=1)]
    modality: Literal["text", "image", "video"] = "text"
    media: str | list[str] | None = None
    sampling: SamplingBody = Field(default_factory=SamplingBody)
    stream: bool = False
    ttft_slo_ms: Annotated[float, Field(gt=0.0, allow_inf_nan=False)] | None = None  # beyond the reference: see GenerationRequest

    @model_validator(mode="after")
    def _check_media(self) -> "GenerateBody":
        if self.modality == "text" and self.media is not None:
            raise ValueError("text requests must not include media")
        if self.modality != "text" and self.media is None:
            raise ValueError(f"{self.modality} requests require media")
        if isinstance(self.media, list) and not self.media:
            raise ValueError("media lists must not be empty")
        if self.modality == "video":
            if not isinstance(self.media, list):
                raise ValueError("video requests require an explicit list of sampled data:image frames")
            if any(not s.startswith("data:image/") for s in self.media):
                raise ValueError("video media lists must contain sampled data:image frame URLs")
        return self


def decode_media(source: str):
    """``data:image/...;base64,...`` -> PIL image; anything else is passed through as a path."""
    if not source.startswith("data:image/"):
        return source
    from PIL import Image

    try:
        header, payload = source.split(",", 1)
        if ";base64" not in header:
            raise ValueError("data URL must be base64 encoded")
        return Image.open(io.BytesIO(base64.b64decode(payload, validate=True))).convert("RGB")
    except Exception as exc:
        raise ValueError(f"invalid image data URL: {exc}") from exc


def to_generation_request(body: GenerateBody) -> GenerationRequest:
    media = None
    if body.media is not None:
        if isinstance(body.media, list):
            media = tuple(_load(decode_media(s)) for s in body.media)
        else:
            media = _load(decode_media(body.media))
    return GenerationRequest(
        request_id=body.request_id or uuid.uuid4().hex, prompt=body.prompt, modality=Modality(body.modality), media=media,
        sampling_params=SamplingParams(temperature=body.sampling.temperature, max_tokens=body.sampling.max_tokens,
                                       ignore_eos=body.sampling.ignore_eos), ttft_slo_ms=body.ttft_slo_ms)


def _load(obj):
    if isinstance(obj, str):
        from PIL import Image

        return Image.open(obj).convert("RGB")
    return obj


def sse(event: ServingEvent) -> bytes:
    return f"event: {event.kind.value}\ndata: {json.dumps(event.to_dict())}\n\n".encode()


async def _stream(runtime: ServingRuntime, handle: RequestHandle, request: Request) -> AsyncIterator[bytes]:
    try:
        while True:
            event = await handle.next_event()
            yield sse(event)
            if event.kind in (EventKind.DONE, EventKind.ERROR):
                return
    finally:
        if not handle.closed:  # the client went away mid-stream
            runtime.cancel(handle.request_id)


async def _collect(handle: RequestHandle) -> ServingEvent:
    while True:
        event = await handle.next_event()
        if event.kind in (EventKind.DONE, EventKind.ERROR):
            return event


async def _disconnected(request: Request) -> None:
    while True:
        message = await request.receive()
        if message["type"] == "http.disconnect":
            return


def prometheus_text(stats: dict[str, float]) -> str:
    """``name -> number`` as Prometheus text format 0.0.4.  Names are sanitised to ``[a-zA-Z0-9_]``; values that only
    grow are still typed ``gauge``, since an engine restart sets them back."""
    lines = []
    for name in sorted(stats):
        value = float(stats[name])
        metric = "prism_" + "".join(ch if ch.isalnum() or ch == "_" else "_" for ch in name)
        shown = "NaN" if value != value else ("+Inf" if value == float("inf") else "-Inf" if value == float("-inf") else repr(value))
        lines += [f"# TYPE {metric} gauge", f"{metric} {shown}"]
    return "\n".join(lines) + "\n"


def create_app(runtime: ServingRuntime, *, manage_runtime: bool = True, model_name: str = "prism") -> FastAPI:
    @asynccontextmanager
    async def lifespan(_: FastAPI) -> AsyncIterator[None]:
        if manage_runtime:
            await asyncio.get_running_loop().run_in_executor(None, runtime.start)
        try:
            yield
        finally:
            if manage_runtime:
                await asyncio.get_running_loop().run_in_executor(None, runtime.stop)

    app = FastAPI(title="prism-serve (B200)", lifespan=lifespan)

    @app.get("/health")
    async def health() -> JSONResponse:
        if runtime.is_healthy:
            restarts = list(getattr(runtime, "restarts", ()))
            return JSONResponse({"status": "ok", **({"restarts": restarts} if restarts else {})})
        detail = str(runtime.failure) if runtime.failure is not None else "engine is not running"
        return JSONResponse({"status": "unavailable", "error": detail}, status_code=503)

    @app.get("/metrics")
    async def metrics():
        """Prometheus text exposition of ``runtime.stats()``: one gauge per name, prefixed ``prism_``."""
        from starlette.responses import PlainTextResponse

        return PlainTextResponse(prometheus_text(runtime.stats()), media_type="text/plain; version=0.0.4; charset=utf-8")

    @app.get("/v1/stats")
    async def stats() -> JSONResponse:
        return JSONResponse(runtime.stats())

    from .openai_api import build_router

    app.include_router(build_router(runtime, model_name, decode_media, _load))  # /v1/chat/completions, /v1/models

    @app.delete("/v1/requests/{request_id}")
    async def cancel(request_id: str) -> JSONResponse:
        """Cancel an open request by the id it was submitted with (beyond the reference, where only a disconnect
        cancels).  The request's own answer or stream ends with ``finish_reason: "cancelled"``."""
        if not runtime.is_open(request_id):
            raise HTTPException(status_code=404, detail=f"no open request {request_id!r}")
        runtime.cancel(request_id)
        return JSONResponse({"request_id": request_id, "status": "cancelling"}, status_code=202)

    @app.post("/v1/generate")
    async def generate(body: GenerateBody, request: Request):
        try:
            gen = to_generation_request(body)
            handle = runtime.submit(gen, asyncio.get_running_loop())
        except IngressFull as exc:
            raise HTTPException(status_code=429, detail=str(exc), headers={"Retry-After": "1"}) from exc
        except RuntimeUnavailable as exc:
            raise HTTPException(status_code=503, detail=str(exc)) from exc
        except DuplicateRequest as exc:
            raise HTTPException(status_code=409, detail=str(exc)) from exc
        except (ValueError, TypeError, OSError) as exc:
            raise HTTPException(status_code=400, detail=str(exc)) from exc
        if body.stream:
            return StreamingResponse(_stream(runtime, handle, request), media_type="text/event-stream")
        result = asyncio.ensure_future(_collect(handle))
        gone = asyncio.ensure_future(_disconnected(request))
        done, _ = await asyncio.wait({result, gone}, return_when=asyncio.FIRST_COMPLETED)
        if result not in done:
            result.cancel()
            runtime.cancel(handle.request_id)
            raise HTTPException(status_code=499, detail="client disconnected")
        gone.cancel()
        event = result.result()
        if event.kind is EventKind.ERROR:
            raise HTTPException(status_code=400, detail=event.error)
        return JSONResponse(event.to_dict())

    return app
