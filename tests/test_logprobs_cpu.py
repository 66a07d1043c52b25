"""Log-probabilities of generated tokens: plain decoding, speculative decoding (one entry per
accepted token), requests cut short by a stop token, and the OpenAI response blocks."""

import math

import pytest

from arcticinference_b200 import LLM, SamplingParams

KW = dict(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64)
PROMPTS = [{"prompt_token_ids": list(range(5, 40))}, {"prompt_token_ids": [7, 8, 9, 7, 8, 9, 7, 8]}]


@pytest.mark.parametrize("spec", [None, {"method": "suffix"}])
def test_every_generated_token_has_its_logprob(spec):
    llm = LLM(speculative_config=spec, **KW)
    sp = [SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True, logprobs=3),
          SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True)]
    a, b = llm.generate(PROMPTS, sp)
    c = a.outputs[0]
    assert len(c.logprobs) == len(c.token_ids) == 24 and len(c.top_logprobs) == 24
    for t, lp, alt in zip(c.token_ids, c.logprobs, c.top_logprobs):
        assert len(alt) == 3 and lp <= 0.0
        # greedy: the chosen token is the most likely one and is listed with the same value
        assert t in alt and math.isclose(alt[t], lp, abs_tol=1e-6) and lp >= max(alt.values()) - 1e-6
    assert math.isclose(c.cumulative_logprob, sum(c.logprobs), rel_tol=1e-9)
    assert b.outputs[0].logprobs is None and b.outputs[0].top_logprobs is None


def test_logprobs_do_not_depend_on_speculation():
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True, logprobs=1)
    plain = LLM(**KW).generate(PROMPTS, sp)
    spec = LLM(speculative_config={"method": "suffix"}, **KW).generate(PROMPTS, sp)
    for x, y in zip(plain, spec):
        assert x.outputs[0].token_ids == y.outputs[0].token_ids
        assert all(math.isclose(p, q, abs_tol=1e-4) for p, q in zip(x.outputs[0].logprobs,
                                                                     y.outputs[0].logprobs))


def test_stop_token_cuts_tokens_and_logprobs_together():
    base = LLM(**KW).generate(PROMPTS[:1], SamplingParams(temperature=0.0, max_tokens=16,
                                                           ignore_eos=True))[0].outputs[0].token_ids
    sp = SamplingParams(temperature=0.0, max_tokens=16, stop_token_ids=[base[5]], logprobs=2)
    for spec in (None, {"method": "suffix"}):
        c = LLM(speculative_config=spec, **KW).generate(PROMPTS[:1], sp)[0].outputs[0]
        assert c.finish_reason == "stop" and len(c.token_ids) <= 6
        assert len(c.logprobs) == len(c.token_ids) == len(c.top_logprobs)


def test_openai_logprob_blocks():
    from fastapi.testclient import TestClient
    from arcticinference_b200.config import EngineArgs
    from arcticinference_b200.engine.async_llm import AsyncLLM
    from arcticinference_b200.entrypoints.openai_server import build_app
    llm = AsyncLLM.from_engine_args(EngineArgs(model="llama-tiny", max_model_len=256,
                                               num_gpu_blocks_override=64), device="cpu").start()
    try:
        with TestClient(build_app(llm, "m")) as c:
            r = c.post("/v1/completions", json={"model": "m", "prompt": "abc", "max_tokens": 5,
                                                "temperature": 0, "ignore_eos": True, "logprobs": 2})
            lp = r.json()["choices"][0]["logprobs"]
            assert len(lp["tokens"]) == len(lp["token_logprobs"]) == len(lp["top_logprobs"]) == 5
            assert all(len(d) >= 1 for d in lp["top_logprobs"])
            r = c.post("/v1/chat/completions", json={
                "model": "m", "max_tokens": 4, "temperature": 0, "ignore_eos": True,
                "messages": [{"role": "user", "content": "hi"}], "logprobs": True, "top_logprobs": 2})
            content = r.json()["choices"][0]["logprobs"]["content"]
            assert len(content) == 4 and all(len(e["top_logprobs"]) == 2 for e in content)
    finally:
        llm.shutdown()
