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
            r = c.post("/v1/completions", json={"model": "m", "prompt": [5, 6, 7, 8, 9], "max_tokens": 2,
                                                "temperature": 0, "prompt_logprobs": 0})
            pl = r.json()["choices"][0]["prompt_logprobs"]
            assert len(pl) == 5 and pl[0] is None and all(v < 0 for v in pl[1:])
            r = c.post("/v1/chat/completions", json={
                "model": "m", "max_tokens": 4, "temperature": 0, "ignore_eos": True,
                "messages": [{"role": "user", "content": "hi"}], "logprobs": True, "top_logprobs": 2})
            content = r.json()["choices"][0]["logprobs"]["content"]
            assert len(content) == 4 and all(len(e["top_logprobs"]) == 2 for e in content)
    finally:
        llm.shutdown()


def test_prompt_logprobs_agree_with_decoding_and_with_chunking():
    prompt = list(range(5, 45))
    llm = LLM(**KW)
    gen = llm.generate([{"prompt_token_ids": prompt}],
                       SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True, logprobs=1))[0]
    toks, lps = gen.outputs[0].token_ids, gen.outputs[0].logprobs
    # teacher forcing: the prompt extended by the generated tokens must score them the same
    sp = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True, prompt_logprobs=0)
    full = llm.generate([{"prompt_token_ids": prompt + toks}, {"prompt_token_ids": [7, 8, 9]}],
                        [sp, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True)])
    pl = full[0].prompt_logprobs
    assert len(pl) == len(prompt) + 4 and pl[0] is None and all(v <= 0 for v in pl[1:])
    for i, want in enumerate(lps):
        assert math.isclose(pl[len(prompt) + i], want, abs_tol=2e-2)      # bf16 model
    assert full[1].prompt_logprobs is None
    # the same prompt in 16-token chunks that share steps with another request's decodes
    chunked = LLM(max_num_batched_tokens=16, **KW).generate(
        [{"prompt_token_ids": prompt + toks}, {"prompt_token_ids": [7, 8, 9]}],
        [sp, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)])
    assert all(math.isclose(a, b, abs_tol=2e-2) for a, b in zip(pl[1:], chunked[0].prompt_logprobs[1:]))
    # with run-ahead stepping on (the default) and off
    off = LLM(async_scheduling=False, max_num_batched_tokens=16, **KW).generate(
        [{"prompt_token_ids": prompt + toks}], sp)[0]
    assert all(math.isclose(a, b, abs_tol=2e-2)
               for a, b in zip(off.prompt_logprobs[1:], chunked[0].prompt_logprobs[1:]))


def test_prompt_logprobs_refused_for_swiftkv():
    llm = LLM(model="llama-tiny-swiftkv", device="cpu", max_model_len=256, num_gpu_blocks_override=64)
    with pytest.raises(ValueError):
        llm.generate([{"prompt_token_ids": [1, 2, 3]}], SamplingParams(prompt_logprobs=0))


def test_prompt_logprobs_are_complete_when_the_prompt_is_in_the_prefix_cache():
    llm = LLM(enable_prefix_caching=True, **KW)
    prompt = [{"prompt_token_ids": list(range(9, 80))}]
    sp = SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True, prompt_logprobs=0)
    first = llm.generate(prompt, sp)[0].prompt_logprobs
    plain = llm.generate(prompt, SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))[0]
    assert plain.num_cached_tokens > 0 and plain.prompt_logprobs is None
    again = llm.generate(prompt, sp)[0].prompt_logprobs
    assert len(again) == 71 and again[0] is None and None not in again[1:]
    assert all(math.isclose(a, b, abs_tol=2e-2) for a, b in zip(first[1:], again[1:]))
