"""OpenAI-compatible proxy that adds Dynasor early exit to a reasoning model's server.

    client --> proxy (this module) --> upstream OpenAI-compatible server

``POST /v1/chat/completions`` and ``POST /v1/completions`` accept one extra body field,
``"dynasor": {"probe_interval": 32, "certainty_window": 3}``; with it the proxy streams the
upstream generation, probes concurrently every ``probe_interval`` chunks and ends the stream
early once the probes agree (see :mod:`.controller`). Without the field, and for every other
path, requests are forwarded unchanged, streaming included
(reference: arctic_inference/dynasor/openai_server.py:190-462).

    python -m arcticinference_b200.dynasor.openai_server --target http://127.0.0.1:8001 --port 8000
"""

from __future__ import annotations

import argparse
import json
import time
import uuid
from contextlib import asynccontextmanager
from typing import AsyncIterator, Optional

import aiohttp
from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .certainty import DEFAULT_PROBE_SUFFIX, format_probe_prompt
from .controller import DynasorController

PROBE_MAX_TOKENS = 32
PROBE_TEMPERATURE = 0.6


async def _sse_objects(resp: aiohttp.ClientResponse) -> AsyncIterator[dict]:
    """Decoded JSON payloads of an SSE response, without the final [DONE]."""
    buf = b""
    async for part in resp.content.iter_any():
        buf += part
        while b"\n\n" in buf:
            event, buf = buf.split(b"\n\n", 1)
            for line in event.split(b"\n"):
                if line.startswith(b"data: "):
                    data = line[6:].strip()
                    if data == b"[DONE]":
                        return
                    try:
                        yield json.loads(data)
                    except json.JSONDecodeError:
                        continue


def build_app(target: str, probe_template: Optional[str] = None) -> FastAPI:
    state = {"session": None}

    @asynccontextmanager
    async def lifespan(_app):
        yield
        if state["session"] is not None:
            await state["session"].close()

    app = FastAPI(title="dynasor proxy", lifespan=lifespan)
    target = target.rstrip("/")

    async def session() -> aiohttp.ClientSession:
        if state["session"] is None:
            state["session"] = aiohttp.ClientSession()
        return state["session"]

    async def upstream_text_stream(path: str, body: dict, chat: bool) -> AsyncIterator[tuple]:
        s = await session()
        async with s.post(target + path, json=dict(body, stream=True)) as resp:
            if resp.status != 200:
                raise RuntimeError("upstream answered %d: %s" % (resp.status, (await resp.text())[:200]))
            async for obj in _sse_objects(resp):
                for ch in obj.get("choices", []):
                    text = (ch.get("delta", {}) or {}).get("content") if chat else ch.get("text")
                    yield text or "", ch.get("finish_reason")

    async def probe(model: str, prompt_text: str, generated: str) -> str:
        s = await session()
        body = {"model": model, "max_tokens": PROBE_MAX_TOKENS, "temperature": PROBE_TEMPERATURE,
                "stream": False,
                "prompt": format_probe_prompt(prompt_text, generated, DEFAULT_PROBE_SUFFIX,
                                              probe_template)}
        async with s.post(target + "/v1/completions", json=body) as resp:
            if resp.status != 200:
                return ""
            data = await resp.json()
            return data["choices"][0].get("text", "") if data.get("choices") else ""

    async def dynasor_stream(path: str, body: dict, chat: bool):
        opts = body.pop("dynasor") or {}
        model = body.get("model", "")
        if chat:
            msgs = body.get("messages", [])
            prompt_text = next((m.get("content", "") for m in reversed(msgs)
                                if m.get("role") == "user"), "")
        else:
            p = body.get("prompt", "")
            prompt_text = p if isinstance(p, str) else ""
        ctl = DynasorController(lambda gen: probe(model, prompt_text, gen),
                                int(opts.get("probe_interval", 32)),
                                int(opts.get("certainty_window", 3)))
        cid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex
        created = int(time.time())
        finish = {"reason": None}

        async def texts():
            async for text, fr in upstream_text_stream(path, body, chat):
                if fr is not None:
                    finish["reason"] = fr
                if text:
                    yield text

        def chunk(text: str, fr=None) -> bytes:
            if chat:
                ch = {"index": 0, "delta": {"content": text}, "finish_reason": fr}
                obj = "chat.completion.chunk"
            else:
                ch = {"index": 0, "text": text, "finish_reason": fr}
                obj = "text_completion"
            return ("data: %s\n\n" % json.dumps({"id": cid, "object": obj, "created": created,
                                                 "model": model, "choices": [ch]})).encode()

        async def gen():
            try:
                async for text in ctl.run(texts()):
                    yield chunk(text)
                st = ctl.stats
                yield chunk("", "stop" if st.early_exit else (finish["reason"] or "stop"))
                yield ("data: %s\n\n" % json.dumps({
                    "id": cid, "object": "dynasor.stats", "choices": [],
                    "dynasor": {"early_exit": st.early_exit, "probes": st.probes,
                                "chunks": st.chunks, "answer": st.answer}})).encode()
            except Exception as e:  # noqa: BLE001 - reported in-band: headers are already sent
                yield ("data: %s\n\n" % json.dumps({"error": {"message": str(e)}})).encode()
            yield b"data: [DONE]\n\n"

        return StreamingResponse(gen(), media_type="text/event-stream")

    async def forward(request: Request, path: str):
        s = await session()
        raw = await request.body()
        headers = {k: v for k, v in request.headers.items()
                   if k.lower() not in ("host", "content-length")}
        stream = False
        if raw:
            try:
                stream = bool(json.loads(raw).get("stream"))
            except (json.JSONDecodeError, AttributeError):
                pass
        url = target + "/" + path.lstrip("/")
        if request.url.query:
            url += "?" + request.url.query
        if stream:
            async def gen():
                async with s.request(request.method, url, data=raw, headers=headers) as resp:
                    async for part in resp.content.iter_any():
                        yield part
            return StreamingResponse(gen(), media_type="text/event-stream")
        async with s.request(request.method, url, data=raw, headers=headers) as resp:
            body = await resp.read()
            return Response(content=body, status_code=resp.status,
                            media_type=resp.headers.get("content-type"))

    async def completions(request: Request, path: str, chat: bool):
        try:
            body = json.loads(await request.body() or b"{}")
        except json.JSONDecodeError:
            return JSONResponse({"error": {"message": "invalid JSON"}}, status_code=400)
        if isinstance(body, dict) and body.get("dynasor") is not None:
            return await dynasor_stream(path, body, chat)
        return await forward(request, path)

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        return await completions(request, "/v1/chat/completions", True)

    @app.post("/v1/completions")
    async def text_completions(request: Request):
        return await completions(request, "/v1/completions", False)

    @app.api_route("/{path:path}", methods=["GET", "POST", "PUT", "DELETE", "PATCH"])
    async def everything_else(request: Request, path: str):
        return await forward(request, path)

    return app


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Dynasor early-exit proxy")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--target", "--target-base-url", dest="target", default="http://127.0.0.1:8001")
    ap.add_argument("--probe-template", default=None,
                    help="format string with {system} {prompt} {generated} {suffix}")
    return ap


def main(argv=None) -> None:
    ns = make_parser().parse_args(argv)
    import uvicorn
    uvicorn.run(build_app(ns.target, ns.probe_template), host=ns.host, port=ns.port)


if __name__ == "__main__":
    main()
