"""Dynasor: answer extraction, math equivalence, the certainty rule, the early-exit loop and
the proxy in front of a scripted upstream server."""

import asyncio
import json
import threading
import time

import pytest
import requests
import uvicorn
from fastapi import FastAPI, Request
from fastapi.responses import StreamingResponse

from arcticinference_b200.dynasor import (DynasorController, count_not_empty, equal_group,
                                          majority_voting, math_equal, obtain_answer,
                                          should_early_exit)
from arcticinference_b200.dynasor.certainty import (format_probe_prompt, formalize_final_response,
                                                    item_entropy)
from arcticinference_b200.dynasor.openai_server import build_app


@pytest.mark.parametrize("a,b,want", [
    ("0.5", "\\frac{1}{2}", True), ("50\\%", "0.5", True), ("1,000", "1000", True), ("(B)", "b", True),
    ("x=5", "5", True), ("\\frac{\\sqrt{3}}{2}", "sqrt(3)/2", True), ("(1,2)", "(1, 2.0)", True),
    ("(1,2)", "[1,2]", False), ("2x+1", "1+2x", True), ("3", "4", False), ("y=2x", "2x-y=0", True),
    ("", "1", False), ("12 \\text{ cm}", "12", True), ("\\dfrac{3}{4}", "0.75", True),
    ("\\begin{pmatrix}1&2\\\\3&4\\end{pmatrix}", "\\begin{pmatrix}1&2\\\\3&4.0\\end{pmatrix}", True),
    ("\\boxed{7}", "7", True), ("A", "B", False), ("1.00005", "1", True), ("1.01", "1", False),
])
def test_math_equal(a, b, want):
    assert math_equal(a, b) is want and math_equal(b, a) is want


def test_answer_extraction_and_certainty_rule():
    assert obtain_answer("42} and more") == "42"
    assert obtain_answer("\\frac{1}{2}} tail") == "\\frac{1}{2}"
    assert obtain_answer("never closes {") == ""
    assert count_not_empty(["", " ", "3", None]) == 1
    assert equal_group(["0.5", "1/2", "\\frac{1}{2}"]) and not equal_group(["1", "2"]) and not equal_group([])
    assert majority_voting(["3", "4", "3.0", ""]) == "3" and majority_voting(["", None]) is None
    assert item_entropy(["1", "1.0", "2"]) == pytest.approx(0.6365, abs=1e-3)
    ok = ["the answer is 4} done"] * 3
    assert should_early_exit(["4", "4.0", "4"], ok, 3)
    assert not should_early_exit(["4", "4"], ok[:2], 3)                      # too few probes
    assert not should_early_exit(["4", "5", "4"], ok, 3)                     # disagreement
    assert not should_early_exit(["4", "", "4"], ok, 3)                      # empty answer
    assert not should_early_exit(["4", "4", "4"], ok[:2] + ["4} wait, no"], 3)   # hesitation
    assert should_early_exit(["9", "4", "4"], ["x"] * 3, 2)                  # window looks back 2 only
    p = format_probe_prompt("Q?", "thinking", "SUFFIX")
    assert "Q?" in p and p.endswith("thinking SUFFIX")
    assert "</think>" in formalize_final_response("no close tag", "4")
    assert "</think>" not in formalize_final_response("done </think>", "4")


def test_controller_exits_early_and_cancels_upstream():
    async def main():
        closed = {"v": False}
        probes = []

        async def chunks():
            try:
                for i in range(1000):
                    yield "t%d " % i
                    await asyncio.sleep(0)
            finally:
                closed["v"] = True

        async def probe(generated):
            probes.append(len(generated.split()))
            n = len(probes)
            return "7} sure" if n >= 3 else "%d} hmm" % n

        ctl = DynasorController(probe, probe_interval=4, certainty_window=2)
        out = [t async for t in ctl.run(chunks())]
        assert ctl.stats.early_exit and ctl.stats.answer == "7" and closed["v"]
        assert "\\boxed{7}" in out[-1] and ctl.stats.probes >= 4 and ctl.stats.chunks < 100
        # a model that never agrees runs to the end
        async def few():
            for i in range(20):
                yield "x "
        ctl2 = DynasorController(lambda g: asyncio.sleep(0, result="%d}" % len(g)), 4, 2)
        out2 = [t async for t in ctl2.run(few())]
        assert len(out2) == 20 and not ctl2.stats.early_exit
    asyncio.run(main())


def _upstream_app():
    app = FastAPI()
    app.state.probes = 0

    @app.get("/v1/models")
    async def models():
        return {"data": [{"id": "fake"}]}

    @app.post("/v1/completions")
    async def completions(request: Request):
        body = await request.json()
        if not body.get("stream"):
            app.state.probes += 1
            return {"choices": [{"text": "12} that is it" if app.state.probes >= 2 else "3} hmm", "index": 0}]}

        async def gen():
            for i in range(400):
                yield "data: %s\n\n" % json.dumps({"choices": [{"index": 0, "text": "w%d " % i, "finish_reason": None}]})
                await asyncio.sleep(0.002)
            yield "data: [DONE]\n\n"
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.post("/v1/chat/completions")
    async def chat(request: Request):
        body = await request.json()

        async def gen():
            for i in range(400):
                yield "data: %s\n\n" % json.dumps({"choices": [{"index": 0, "delta": {"content": "w%d " % i},
                                                                 "finish_reason": None}]})
                await asyncio.sleep(0.002)
            yield "data: [DONE]\n\n"
        if body.get("stream"):
            return StreamingResponse(gen(), media_type="text/event-stream")
        return {"choices": [{"index": 0, "message": {"role": "assistant", "content": "plain"}}]}
    return app


def _serve(app, port):
    cfg = uvicorn.Config(app, host="127.0.0.1", port=port, log_level="warning")
    srv = uvicorn.Server(cfg)
    th = threading.Thread(target=srv.run, daemon=True)
    th.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    return srv, th


def test_proxy_end_to_end():
    up, t1 = _serve(_upstream_app(), 18431)
    px, t2 = _serve(build_app("http://127.0.0.1:18431"), 18432)
    try:
        base = "http://127.0.0.1:18432"
        assert requests.get(base + "/v1/models").json() == {"data": [{"id": "fake"}]}          # forwarded
        plain = requests.post(base + "/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}]})
        assert plain.json()["choices"][0]["message"]["content"] == "plain"
        body = {"model": "fake", "messages": [{"role": "user", "content": "What is 3*4?"}], "stream": True,
                "dynasor": {"probe_interval": 8, "certainty_window": 2}}
        texts, stats = [], None
        with requests.post(base + "/v1/chat/completions", json=body, stream=True) as r:
            for line in r.iter_lines():
                if line.startswith(b"data: {"):
                    obj = json.loads(line[6:])
                    if obj.get("object") == "dynasor.stats":
                        stats = obj["dynasor"]
                    for ch in obj.get("choices", []):
                        texts.append((ch.get("delta") or {}).get("content") or "")
        full = "".join(texts)
        assert stats["early_exit"] and stats["answer"] == "12" and stats["chunks"] < 400
        assert "\\boxed{12}" in full and full.startswith("w0 w1 ")
        # text-completions flavour, forwarded stream when the field is absent
        with requests.post(base + "/v1/completions", json={"prompt": "p", "stream": True}, stream=True) as r:
            n = sum(1 for line in r.iter_lines() if line.startswith(b"data: {"))
        assert n == 400
    finally:
        px.should_exit = True
        up.should_exit = True
        t2.join(5)
        t1.join(5)
