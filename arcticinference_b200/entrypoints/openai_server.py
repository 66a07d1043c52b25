"""OpenAI-compatible HTTP server on top of :class:`AsyncLLM`.

The reference is reached through ``vllm serve`` with its extra flags
(``--ulysses-sequence-parallel-size``, ``--enable-shift-parallel``, ``--speculative-config``;
README.md:98-124) and its clients (benchmarks, Dynasor) speak the OpenAI completions and
chat-completions protocols, streaming included. This module provides those routes:

    GET  /health  /v1/models  /metrics  /version
    POST /v1/completions  /v1/chat/completions  /tokenize  /detokenize
    POST /sleep?level=1  /wake_up  /reset_prefix_cache      (development endpoints)
"""

from __future__ import annotations

import json
import time
import uuid
from typing import Any, Optional, Union

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse
from pydantic import BaseModel

from ..engine.async_llm import AsyncLLM
from ..engine.sampling_params import SamplingParams
from ..utils.tokenizer import chat_token_ids


class CompletionRequest(BaseModel):
    model: Optional[str] = None
    prompt: Union[str, list[str], list[int], list[list[int]]]
    max_tokens: Optional[int] = 16
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[dict[str, float]] = None
    include_stop_str_in_output: bool = False
    skip_special_tokens: bool = True
    n: int = 1
    stream: bool = False
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    seed: Optional[int] = None
    logprobs: Optional[int] = None
    echo: bool = False
    ignore_eos: bool = False
    min_tokens: int = 0
    max_tokens_n: Optional[list[int]] = None
    prompt_logprobs: Optional[int] = None     # also score the prompt tokens
    guided_choice: Optional[list[str]] = None   # the completion is exactly one of these
    guided_json: Optional[Union[dict, str]] = None   # compact JSON conforming to this schema
    guided_regex: Optional[str] = None              # the completion matches this expression
    response_format: Optional[dict] = None
    routing_key: Optional[str] = None


class ChatMessage(BaseModel):
    role: str
    content: Union[str, list[dict], None] = ""


class ChatCompletionRequest(BaseModel):
    model: Optional[str] = None
    messages: list[ChatMessage]
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[dict[str, float]] = None
    include_stop_str_in_output: bool = False
    skip_special_tokens: bool = True
    n: int = 1
    stream: bool = False
    stop: Optional[Union[str, list[str]]] = None
    stop_token_ids: Optional[list[int]] = None
    seed: Optional[int] = None
    logprobs: Optional[bool] = None
    top_logprobs: Optional[int] = None
    ignore_eos: bool = False
    add_generation_prompt: bool = True
    continue_final_message: bool = False
    routing_key: Optional[str] = None
    guided_choice: Optional[list[str]] = None
    guided_json: Optional[Union[dict, str]] = None
    guided_regex: Optional[str] = None
    response_format: Optional[dict] = None


class TokenizeRequest(BaseModel):
    model: Optional[str] = None
    prompt: Optional[str] = None
    messages: Optional[list[ChatMessage]] = None
    add_special_tokens: bool = True


class DetokenizeRequest(BaseModel):
    model: Optional[str] = None
    tokens: list[int]


def _schema_of(req):
    """JSON schema asked for by ``guided_json`` or by an OpenAI ``response_format`` of type
    ``json_schema`` (``{"type": "json_schema", "json_schema": {"schema": {...}}}``)."""
    if getattr(req, "guided_json", None) is not None:
        return req.guided_json
    rf = getattr(req, "response_format", None)
    if rf and rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return js.get("schema", js) or None
    return None


def _checked_schema(req):
    """The request's schema, compiled once here so that an unsupported one is a client error
    (ValueError) instead of a failure inside the engine loop."""
    schema = _schema_of(req)
    if schema is not None:
        from ..structured.json_schema import compile_schema
        compile_schema(schema)
    return schema


def _checked_regex(req):
    pattern = getattr(req, "guided_regex", None)
    if pattern is not None:
        from ..structured.regex import compile_regex
        compile_regex(pattern)
    return pattern


def _sampling(req, max_tokens) -> SamplingParams:
    lp = getattr(req, "top_logprobs", None) if isinstance(req, ChatCompletionRequest) and req.logprobs \
        else (req.logprobs if not isinstance(req, ChatCompletionRequest) else None)
    return SamplingParams(n=req.n, temperature=req.temperature, top_p=req.top_p, top_k=req.top_k,
                          min_p=req.min_p, presence_penalty=req.presence_penalty,
                          frequency_penalty=req.frequency_penalty,
                          repetition_penalty=req.repetition_penalty, logit_bias=req.logit_bias,
                          include_stop_str_in_output=req.include_stop_str_in_output,
                          skip_special_tokens=req.skip_special_tokens,
                          max_tokens=max_tokens, stop=req.stop, stop_token_ids=req.stop_token_ids,
                          seed=req.seed, logprobs=lp, ignore_eos=req.ignore_eos,
                          prompt_logprobs=getattr(req, "prompt_logprobs", None),
                          min_tokens=getattr(req, "min_tokens", 0),
                          max_tokens_n=getattr(req, "max_tokens_n", None),
                          guided_choice=getattr(req, "guided_choice", None) or None,
                          guided_json=_checked_schema(req), guided_regex=_checked_regex(req))


def _sse(obj: Any) -> str:
    return "data: %s\n\n" % json.dumps(obj)


def _message_text(m: ChatMessage) -> str:
    if isinstance(m.content, list):
        return "".join(p.get("text", "") for p in m.content if isinstance(p, dict))
    return m.content or ""


def build_app(llm: AsyncLLM, served_model_name: Optional[str] = None) -> FastAPI:
    app = FastAPI(title="arcticinference_b200")
    name = served_model_name or llm.engine.config.model.name_or_path or "model"
    tok = llm.engine.tokenizer
    started = time.time()

    def check_model(m: Optional[str]) -> None:
        if m and m != name:
            raise HTTPException(status_code=404, detail="model %r is not served (serving %r)" % (m, name))

    def chat_prompt_ids(req) -> list:
        msgs = [{"role": m.role, "content": _message_text(m)} for m in req.messages]
        extra = {}
        if getattr(req, "continue_final_message", False):
            # the last message is a partial assistant turn that the model goes on writing
            if getattr(req, "add_generation_prompt", True) and "add_generation_prompt" in req.model_fields_set:
                raise HTTPException(status_code=400, detail="continue_final_message and "
                                    "add_generation_prompt exclude each other")
            extra["continue_final_message"] = True
            return chat_token_ids(tok, msgs, False, **extra)
        return chat_token_ids(tok, msgs, getattr(req, "add_generation_prompt", True))

    # ------------------------------------------------------------------ plumbing
    @app.get("/health")
    async def health():
        if llm._dead is not None:
            raise HTTPException(status_code=503, detail="engine loop died")
        return {"status": "ok"}

    @app.get("/version")
    async def version():
        from .. import __version__
        return {"version": __version__}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": name, "object": "model", "created": int(started),
                                            "owned_by": "arcticinference_b200",
                                            "max_model_len": llm.engine.config.scheduler.max_model_len}]}

    @app.get("/metrics")
    async def metrics():
        s = await llm.get_stats()
        lines = []
        for key, help_, typ in (
                ("prompt_tokens", "prompt tokens processed", "counter"),
                ("generation_tokens", "tokens generated", "counter"),
                ("steps", "engine steps", "counter"),
                ("draft_tokens", "speculative tokens proposed", "counter"),
                ("accepted_tokens", "speculative tokens accepted", "counter"),
                ("running", "requests running", "gauge"),
                ("waiting", "requests waiting", "gauge"),
                ("kv_cache_usage", "fraction of KV-cache blocks in use", "gauge")):
            lines.append("# HELP arctic_%s %s" % (key, help_))
            lines.append("# TYPE arctic_%s %s" % (key, typ))
            lines.append('arctic_%s{model_name="%s"} %s' % (key, name, s.get(key, 0)))
        for key, help_ in (("drafted_per_position", "drafts that reached this position"),
                           ("accepted_per_position", "drafts accepted at this position")):
            lines.append("# HELP arctic_%s %s" % (key, help_))
            lines.append("# TYPE arctic_%s counter" % key)
            for i, v in enumerate(s.get(key, [])):
                lines.append('arctic_%s{model_name="%s",position="%d"} %s' % (key, name, i, v))
        for key, help_ in (("sp_steps", "steps run in sequence-parallel mode"),
                           ("tp_steps", "steps run in tensor-parallel mode"),
                           ("run_ahead_steps", "steps queued while their predecessor ran"),
                           ("comm_timeouts", "device-side waits that ran out")):
            lines.append("# HELP arctic_%s %s" % (key, help_))
            lines.append("# TYPE arctic_%s counter" % key)
            lines.append('arctic_%s{model_name="%s"} %s' % (key, name, s.get(key, 0)))
        return PlainTextResponse("\n".join(lines) + "\n")

    @app.post("/tokenize")
    async def tokenize(req: TokenizeRequest):
        ids = chat_prompt_ids(req) if req.messages else tok.encode(req.prompt or "")
        ids = list(ids["input_ids"]) if isinstance(ids, dict) else list(ids)
        return {"tokens": ids, "count": len(ids),
                "max_model_len": llm.engine.config.scheduler.max_model_len}

    @app.post("/detokenize")
    async def detokenize(req: DetokenizeRequest):
        return {"prompt": tok.decode(req.tokens)}

    @app.post("/sleep")
    async def sleep(level: int = 1):
        await llm.sleep(level)
        return {"status": "sleeping", "level": level}

    @app.post("/wake_up")
    async def wake_up(request: Request):
        tags = request.query_params.getlist("tags") or None
        await llm.wake_up(tags)
        return {"status": "awake", "tags": tags}

    @app.post("/reset_prefix_cache")
    async def reset_prefix_cache():
        await llm.reset_prefix_cache()
        return {"status": "ok"}

    # ------------------------------------------------------------------ completions
    def usage(prompt_tokens: int, completion_tokens: int) -> dict:
        return {"prompt_tokens": prompt_tokens, "completion_tokens": completion_tokens,
                "total_tokens": prompt_tokens + completion_tokens}

    def logprob_block(comp, chat: bool):
        if comp.logprobs is None:
            return None
        tops = comp.top_logprobs or [{} for _ in comp.token_ids]
        if chat:
            return {"content": [{"token": tok.decode([t]), "logprob": lp,
                                 "top_logprobs": [{"token": tok.decode([int(i)]), "logprob": v}
                                                  for i, v in alt.items()]}
                                for t, lp, alt in zip(comp.token_ids, comp.logprobs, tops)]}
        return {"tokens": [tok.decode([t]) for t in comp.token_ids],
                "token_logprobs": list(comp.logprobs),
                "top_logprobs": [{tok.decode([int(i)]): v for i, v in alt.items()} for alt in tops],
                "text_offset": None}

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest):
        check_model(req.model)
        p = req.prompt
        if isinstance(p, str):
            prompts = [p]
        elif p and isinstance(p[0], int):
            prompts = [p]
        else:
            prompts = list(p)
        if not prompts:
            raise HTTPException(status_code=400, detail="empty prompt")
        try:
            params = _sampling(req, req.max_tokens)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        cid = "cmpl-" + uuid.uuid4().hex
        created = int(time.time())

        if req.stream:
            if len(prompts) != 1:
                raise HTTPException(status_code=400, detail="streaming takes one prompt")

            async def gen():
                sent = {}
                async for out in llm.generate(prompts[0], params, cid, req.routing_key):
                    for c in out.outputs:
                        prev = sent.get(c.index, 0)
                        delta = c.text[prev:]
                        sent[c.index] = len(c.text)
                        if delta or c.finish_reason:
                            yield _sse({"id": cid, "object": "text_completion", "created": created,
                                        "model": name,
                                        "choices": [{"index": c.index, "text": delta,
                                                     "finish_reason": c.finish_reason,
                                                     "logprobs": None}]})
                    if out.finished:
                        n_out = sum(len(c.token_ids) for c in out.outputs)
                        yield _sse({"id": cid, "object": "text_completion", "created": created,
                                    "model": name, "choices": [],
                                    "usage": usage(len(out.prompt_token_ids), n_out)})
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")

        import asyncio
        outs = await asyncio.gather(*[llm.generate_final(pr, params, "%s-%d" % (cid, i), req.routing_key)
                                      for i, pr in enumerate(prompts)])
        choices, n_in, n_out = [], 0, 0
        for i, out in enumerate(outs):
            if out is None:
                raise HTTPException(status_code=499, detail="request aborted")
            n_in += len(out.prompt_token_ids)
            for c in out.outputs:
                n_out += len(c.token_ids)
                text = c.text
                if req.echo:
                    text = (out.prompt if out.prompt is not None else tok.decode(out.prompt_token_ids)) + text
                choices.append({"index": i * req.n + c.index, "text": text, "token_ids": c.token_ids,
                                "finish_reason": c.finish_reason, "logprobs": logprob_block(c, False)})
                if req.prompt_logprobs is not None:
                    choices[-1]["prompt_logprobs"] = out.prompt_logprobs
        return JSONResponse({"id": cid, "object": "text_completion", "created": created, "model": name,
                             "choices": choices, "usage": usage(n_in, n_out)})

    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatCompletionRequest):
        check_model(req.model)
        if not req.messages:
            raise HTTPException(status_code=400, detail="no messages")
        ids = chat_prompt_ids(req)
        max_tokens = req.max_completion_tokens or req.max_tokens
        if max_tokens is None:
            max_tokens = max(1, llm.engine.config.scheduler.max_model_len - len(ids))
        try:
            params = _sampling(req, max_tokens)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        cid = "chatcmpl-" + uuid.uuid4().hex
        created = int(time.time())

        if req.stream:
            async def gen():
                sent = {}
                first = True
                async for out in llm.generate(ids, params, cid, req.routing_key):
                    for c in out.outputs:
                        prev = sent.get(c.index, 0)
                        delta = c.text[prev:]
                        sent[c.index] = len(c.text)
                        d = {"content": delta}
                        if first:
                            d["role"] = "assistant"
                            first = False
                        if delta or c.finish_reason:
                            yield _sse({"id": cid, "object": "chat.completion.chunk", "created": created,
                                        "model": name,
                                        "choices": [{"index": c.index, "delta": d,
                                                     "finish_reason": c.finish_reason}]})
                    if out.finished:
                        n_out = sum(len(c.token_ids) for c in out.outputs)
                        yield _sse({"id": cid, "object": "chat.completion.chunk", "created": created,
                                    "model": name, "choices": [],
                                    "usage": usage(len(out.prompt_token_ids), n_out)})
                yield "data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")

        out = await llm.generate_final(ids, params, cid, req.routing_key)
        if out is None:
            raise HTTPException(status_code=499, detail="request aborted")
        choices = [{"index": c.index, "message": {"role": "assistant", "content": c.text},
                    "finish_reason": c.finish_reason, "logprobs": logprob_block(c, True)}
                   for c in out.outputs]
        n_out = sum(len(c.token_ids) for c in out.outputs)
        return JSONResponse({"id": cid, "object": "chat.completion", "created": created, "model": name,
                             "choices": choices, "usage": usage(len(out.prompt_token_ids), n_out)})

    return app
