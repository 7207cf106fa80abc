"""``POST /v1/chat/completions`` and ``GET /v1/models`` in the shape OpenAI-style clients expect, on top of the same
runtime as ``/v1/generate``.  The reference has no such endpoint; this is a thin translation, not a second engine path.

What is translated: one user turn (a string, or parts of type ``text`` and ``image_url`` with ``data:image/...`` URLs
or file paths on the server), optionally preceded by one system message, whose text is put before the user's;
``max_tokens`` / ``max_completion_tokens``, ``temperature``, ``stream``.  Other fields a client sends are ignored.
Conversations of several turns are refused with 400: the engine's chat prompt has one user turn, and silently
flattening a history would change what the model sees.  Streaming answers are ``chat.completion.chunk`` frames
(``data: {...}``) ending with ``data: [DONE]``.
"""

from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, AsyncIterator

from fastapi import APIRouter, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse
from pydantic import BaseModel, ConfigDict, Field

from ..sampling_params import SamplingParams
from .protocol import EventKind, GenerationRequest, Modality
from .runtime import DuplicateRequest, IngressFull, RuntimeUnavailable, ServingRuntime

FINISH = {"eos": "stop", "length": "length"}  # other reasons (cancelled, rejected, shutdown) pass through by name


class ChatMessage(BaseModel):
    model_config = ConfigDict(extra="ignore")
    role: str
    content: str | list[dict[str, Any]]


class ChatBody(BaseModel):
    model_config = ConfigDict(extra="ignore")
    model: str | None = None
    messages: list[ChatMessage] = Field(min_length=1)
    max_tokens: int | None = Field(default=None, gt=0)
    max_completion_tokens: int | None = Field(default=None, gt=0)
    temperature: float = Field(default=0.0, ge=0.0)
    stream: bool = False


def _parts(content: str | list[dict[str, Any]]) -> tuple[str, list[str]]:
    if isinstance(content, str):
        return content, []
    texts, images = [], []
    for part in content:
        kind = part.get("type")
        if kind == "text":
            texts.append(str(part.get("text", "")))
        elif kind == "image_url":
            url = part.get("image_url")
            url = url.get("url") if isinstance(url, dict) else url
            if not isinstance(url, str) or not url:
                raise ValueError("image_url parts need a url")
            images.append(url)
        else:
            raise ValueError(f"unsupported content part type {kind!r}; supported: text, image_url")
    return "\n".join(t for t in texts if t), images


def to_generation_request(body: ChatBody, decode_media, load_media) -> GenerationRequest:
    """``decode_media`` / ``load_media``: the ``/v1/generate`` helpers (data URL -> image, path -> image)."""
    system = [m for m in body.messages if m.role == "system"]
    users = [m for m in body.messages if m.role == "user"]
    others = [m for m in body.messages if m.role not in ("system", "user")]
    if others or len(users) != 1 or len(system) > 1 or body.messages[-1].role != "user":
        raise ValueError("one user message, optionally after one system message, is supported; conversations of several turns are not")
    text, images = _parts(users[0].content)
    if system:
        sys_text, sys_images = _parts(system[0].content)
        if sys_images:
            raise ValueError("images belong to the user message")
        text = f"{sys_text}\n\n{text}" if sys_text else text
    if not text:
        raise ValueError("the user message has no text")
    media = tuple(load_media(decode_media(u)) for u in images) if images else None
    sp = SamplingParams(temperature=body.temperature, max_tokens=body.max_completion_tokens or body.max_tokens or 256)
    return GenerationRequest(request_id=uuid.uuid4().hex, prompt=text, modality=Modality.IMAGE if images else Modality.TEXT,
                             media=media if media is None or len(media) > 1 else media[0], sampling_params=sp)


def _envelope(rid: str, model: str, created: int, kind: str, choice: dict[str, Any], **extra: Any) -> dict[str, Any]:
    return {"id": f"chatcmpl-{rid}", "object": kind, "created": created, "model": model, "choices": [choice], **extra}


def build_router(runtime: ServingRuntime, model_name: str, decode_media, load_media) -> APIRouter:
    router = APIRouter()

    @router.get("/v1/models")
    async def models() -> JSONResponse:
        return JSONResponse({"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "prism-serve"}]})

    @router.post("/v1/chat/completions")
    async def chat(body: ChatBody, request: Request):
        model = body.model or model_name
        try:
            gen = to_generation_request(body, decode_media, load_media)
            handle = runtime.submit(gen, asyncio.get_running_loop())
        except IngressFull as exc:
            raise HTTPException(status_code=429, detail=str(exc), headers={"Retry-After": "1"}) from exc
        except RuntimeUnavailable as exc:
            raise HTTPException(status_code=503, detail=str(exc)) from exc
        except DuplicateRequest as exc:
            raise HTTPException(status_code=409, detail=str(exc)) from exc
        except (ValueError, TypeError, OSError) as exc:
            raise HTTPException(status_code=400, detail=str(exc)) from exc
        created, rid = int(time.time()), gen.request_id

        if body.stream:
            async def frames() -> AsyncIterator[bytes]:
                def frame(delta: dict[str, Any], finish: str | None = None) -> bytes:
                    chunk = _envelope(rid, model, created, "chat.completion.chunk", {"index": 0, "delta": delta, "finish_reason": finish})
                    return f"data: {json.dumps(chunk)}\n\n".encode()

                try:
                    yield frame({"role": "assistant", "content": ""})
                    while True:
                        event = await handle.next_event()
                        if event.kind is EventKind.TOKEN:
                            yield frame({"content": event.token_text or ""})
                        elif event.kind is EventKind.DONE:
                            yield frame({}, FINISH.get(event.finish_reason or "", event.finish_reason))
                            yield b"data: [DONE]\n\n"
                            return
                        elif event.kind is EventKind.ERROR:
                            yield f"data: {json.dumps({'error': {'message': event.error, 'type': 'engine_error'}})}\n\n".encode()
                            yield b"data: [DONE]\n\n"
                            return
                finally:
                    if not handle.closed:  # the client went away mid-stream
                        runtime.cancel(handle.request_id)

            return StreamingResponse(frames(), media_type="text/event-stream")

        async def collect():
            while True:
                event = await handle.next_event()
                if event.kind in (EventKind.DONE, EventKind.ERROR):
                    return event

        async def disconnected():
            while True:
                if (await request.receive())["type"] == "http.disconnect":
                    return

        result, gone = asyncio.ensure_future(collect()), asyncio.ensure_future(disconnected())
        done, _ = await asyncio.wait({result, gone}, return_when=asyncio.FIRST_COMPLETED)
        if result not in done:
            result.cancel()
            runtime.cancel(handle.request_id)
            raise HTTPException(status_code=499, detail="client disconnected")
        gone.cancel()
        event = result.result()
        if event.kind is EventKind.ERROR:
            raise HTTPException(status_code=400, detail=event.error)
        choice = {"index": 0, "message": {"role": "assistant", "content": event.text or ""},
                  "finish_reason": FINISH.get(event.finish_reason or "", event.finish_reason)}
        usage = {"completion_tokens": len(event.token_ids)}
        if event.prompt_tokens is not None:
            usage.update(prompt_tokens=event.prompt_tokens, total_tokens=event.prompt_tokens + len(event.token_ids))
        return JSONResponse(_envelope(rid, model, created, "chat.completion", choice, usage=usage))

    return router
