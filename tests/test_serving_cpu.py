"""AsyncLLM and the OpenAI-compatible server on CPU (tiny random model)."""

import asyncio
import json

import pytest
from fastapi.testclient import TestClient

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import EngineArgs
from arcticinference_b200.engine.async_llm import AsyncLLM, EngineDeadError
from arcticinference_b200.entrypoints.openai_server import build_app

KW = dict(model="llama-tiny", device="cpu", num_gpu_blocks_override=128, block_size=16,
          max_model_len=256, enable_sleep_mode=True)
SP = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
PROMPTS = [[5, 9, 200, 17, 3], [77] * 20, [1, 2, 3]]


@pytest.fixture(scope="module")
def async_llm():
    kw = dict(KW)
    dev = kw.pop("device")
    a = AsyncLLM.from_engine_args(EngineArgs(**kw), device=dev).start()
    yield a
    a.shutdown()


@pytest.fixture(scope="module")
def offline_tokens():
    return [o.outputs[0].token_ids for o in LLM(**KW).generate(PROMPTS, SP)]


def test_streaming_matches_offline(async_llm, offline_tokens):
    async def one(p):
        seen = []
        async for out in async_llm.generate(p, SP):
            seen.append((len(out.outputs[0].token_ids), out.finished))
        return out, seen

    async def run():
        return await asyncio.gather(*[one(p) for p in PROMPTS])

    for (out, seen), want in zip(asyncio.run(run()), offline_tokens):
        assert out.finished and out.outputs[0].token_ids == want
        assert out.outputs[0].finish_reason == "length"
        lens = [n for n, _ in seen]
        assert lens == sorted(lens) and len(seen) >= 2          # several partial outputs
        assert [f for _, f in seen].count(True) == 1


def test_abort_and_parallel_samples(async_llm):
    async def run():
        got = []
        agen = async_llm.generate([4, 5, 6], SamplingParams(temperature=0.0, max_tokens=200,
                                                            ignore_eos=True), "abort-me")
        async for out in agen:
            got.append(out)
            if len(got) == 2:
                await async_llm.abort("abort-me")
        assert not got[-1].finished and len(got[-1].outputs[0].token_ids) < 200
        final = await async_llm.generate_final([9, 9, 9], SamplingParams(
            temperature=0.8, seed=3, n=3, max_tokens=6, ignore_eos=True))
        assert final.finished and [c.index for c in final.outputs] == [0, 1, 2]
        assert all(len(c.token_ids) == 6 for c in final.outputs)
        stats = await async_llm.get_stats()
        assert stats["running"] == 0 and stats["waiting"] == 0
    asyncio.run(run())


def test_sleep_wake_and_errors(async_llm, offline_tokens):
    async def run():
        await async_llm.sleep(2)
        assert (await async_llm.get_stats())["sleeping_level"] == 2
        await async_llm.wake_up()
        out = await async_llm.generate_final(PROMPTS[0], SP)
        assert out.outputs[0].token_ids == offline_tokens[0]
        await async_llm.reset_prefix_cache()
        with pytest.raises(ValueError):
            await async_llm._call("no-such-call")
        assert await async_llm.apply(lambda eng, k: eng.config.model.vocab_size + k, 1) > 1
    asyncio.run(run())


def test_openai_routes(async_llm, offline_tokens):
    client = TestClient(build_app(async_llm, "tiny"))
    assert client.get("/health").json() == {"status": "ok"}
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    body = {"model": "tiny", "prompt": PROMPTS[0], "max_tokens": 12, "temperature": 0, "ignore_eos": True}
    r = client.post("/v1/completions", json=body).json()
    assert r["choices"][0]["token_ids"] == offline_tokens[0]
    assert r["usage"] == {"prompt_tokens": 5, "completion_tokens": 12, "total_tokens": 17}
    # the OpenAI sampling fields reach the sampler: a bias forces the token, a frequency
    # penalty forbids repeats, zeros (what client libraries send by default) change nothing
    r = client.post("/v1/completions", json=dict(body, logit_bias={"77": 100})).json()
    assert r["choices"][0]["token_ids"] == [77] * 12
    r = client.post("/v1/completions", json=dict(body, frequency_penalty=100.0)).json()
    assert len(set(r["choices"][0]["token_ids"])) == 12
    r = client.post("/v1/completions", json=dict(body, presence_penalty=0, frequency_penalty=0)).json()
    assert r["choices"][0]["token_ids"] == offline_tokens[0]
    assert client.post("/v1/completions", json=dict(body, min_p=2.0)).status_code == 400
    # batch of prompts, n samples
    r = client.post("/v1/completions", json=dict(body, prompt=[PROMPTS[0], PROMPTS[2]], n=2,
                                                 temperature=0.5, seed=1)).json()
    assert sorted(c["index"] for c in r["choices"]) == [0, 1, 2, 3]
    # streaming: concatenated deltas equal the non-streamed text
    whole = client.post("/v1/completions", json=body).json()["choices"][0]["text"]
    with client.stream("POST", "/v1/completions", json=dict(body, stream=True)) as resp:
        chunks = [l[6:] for l in resp.iter_lines() if l.startswith("data: ")]
    assert chunks[-1] == "[DONE]"
    parts = [json.loads(c) for c in chunks[:-1]]
    assert "".join(p["choices"][0]["text"] for p in parts if p["choices"]) == whole
    assert parts[-1]["usage"]["completion_tokens"] == 12
    # chat
    chat = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5,
            "temperature": 0, "ignore_eos": True}
    r = client.post("/v1/chat/completions", json=chat).json()
    assert r["choices"][0]["message"]["role"] == "assistant" and r["usage"]["completion_tokens"] == 5
    with client.stream("POST", "/v1/chat/completions", json=dict(chat, stream=True)) as resp:
        chunks = [json.loads(l[6:]) for l in resp.iter_lines() if l.startswith("data: {")]
    assert chunks[0]["choices"][0]["delta"].get("role") == "assistant"
    # an open assistant turn: the model continues it (no generation prompt is appended)
    open_turn = dict(chat, messages=chat["messages"] + [{"role": "assistant", "content": "So"}])
    closed = client.post("/v1/chat/completions", json=open_turn).json()["usage"]["prompt_tokens"]
    cont = client.post("/v1/chat/completions", json=dict(open_turn, continue_final_message=True))
    assert cont.status_code == 200 and cont.json()["usage"]["prompt_tokens"] < closed
    assert client.post("/v1/chat/completions", json=dict(open_turn, continue_final_message=True,
                                                         add_generation_prompt=True)).status_code == 400
    # plumbing
    t = client.post("/tokenize", json={"prompt": "abc"}).json()
    assert client.post("/detokenize", json={"tokens": t["tokens"]}).json()["prompt"] == "abc"
    assert "arctic_generation_tokens" in client.get("/metrics").text
    assert client.post("/v1/completions", json=dict(body, model="other")).status_code == 404
    assert client.post("/v1/completions", json=dict(body, temperature=-1)).status_code == 400
    assert client.post("/sleep?level=1").json()["status"] == "sleeping"
    assert client.post("/wake_up").json()["status"] == "awake"
    assert client.post("/reset_prefix_cache").status_code == 200


def test_cli_parser_takes_arctic_flags():
    from arcticinference_b200.cli import make_parser
    ns = make_parser().parse_args(["serve", "llama-tiny", "--ulysses-sequence-parallel-size", "2",
                                   "--enable-shift-parallel", "--shift-parallel-threshold", "64",
                                   "--speculative-config", '{"method": "suffix"}', "--port", "9000"])
    args = EngineArgs.from_cli_args(ns)
    assert args.ulysses_sequence_parallel_size == 2 and args.enable_shift_parallel
    assert args.shift_parallel_threshold == 64 and ns.port == 9000


def test_dead_engine_reports(async_llm):
    kw = dict(KW)
    dev = kw.pop("device")
    a = AsyncLLM.from_engine_args(EngineArgs(**kw), device=dev).start()
    a.shutdown()

    async def run():
        with pytest.raises(EngineDeadError):
            await a.generate_final([1, 2], SP)
    asyncio.run(run())


def test_guided_choice_over_http(async_llm):
    from fastapi.testclient import TestClient
    from arcticinference_b200.entrypoints.openai_server import build_app
    with TestClient(build_app(async_llm, "m")) as c:
        r = c.post("/v1/completions", json={"model": "m", "prompt": "pick one:", "max_tokens": 16,
                                            "temperature": 0.8, "seed": 1,
                                            "guided_choice": ["red", "green", "blue"]})
        assert r.status_code == 200, r.text
        ch = r.json()["choices"][0]
        assert ch["text"] in ("red", "green", "blue") and ch["finish_reason"] == "stop"
        r = c.post("/v1/chat/completions", json={"model": "m", "max_tokens": 16,
                                                 "messages": [{"role": "user", "content": "?"}],
                                                 "guided_choice": ["yes", "no"]})
        assert r.json()["choices"][0]["message"]["content"] in ("yes", "no")


def test_json_schema_response_format_over_http(async_llm):
    import json
    from fastapi.testclient import TestClient
    from arcticinference_b200.entrypoints.openai_server import build_app
    schema = {"type": "object", "properties": {"answer": {"type": "integer"},
                                               "unit": {"enum": ["m", "s"]}}}
    with TestClient(build_app(async_llm, "m")) as c:
        r = c.post("/v1/chat/completions", json={
            "model": "m", "max_tokens": 64, "temperature": 0.7, "seed": 5,
            "messages": [{"role": "user", "content": "how far?"}],
            "response_format": {"type": "json_schema",
                                "json_schema": {"name": "a", "schema": schema}}})
        assert r.status_code == 200, r.text
        doc = json.loads(r.json()["choices"][0]["message"]["content"])
        assert isinstance(doc["answer"], int) and doc["unit"] in ("m", "s")
        r = c.post("/v1/completions", json={"model": "m", "prompt": "x", "max_tokens": 64,
                                            "guided_json": schema})
        assert set(json.loads(r.json()["choices"][0]["text"])) == {"answer", "unit"}
        r = c.post("/v1/completions", json={"model": "m", "prompt": "x", "max_tokens": 8,
                                            "guided_json": {"type": "string", "pattern": "a"}})
        assert r.status_code >= 400
        r = c.post("/v1/completions", json={"model": "m", "prompt": "x", "max_tokens": 24,
                                            "temperature": 0.9, "seed": 2,
                                            "guided_regex": "[A-C]{2}-[0-9]{3}"})
        import re
        assert re.fullmatch("[A-C]{2}-[0-9]{3}", r.json()["choices"][0]["text"])
        assert c.post("/v1/completions", json={"model": "m", "prompt": "x",
                                               "guided_regex": "(unclosed"}).status_code == 400
