"""Engine options that have no test elsewhere: the fp32 LM head (flag and environment
switch) and per-sample forced lengths for rollout replay."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import EngineArgs

KW = dict(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16, max_model_len=128)


def _greedy(llm, n=8):
    sp = SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)
    return llm.generate([[7, 8, 9, 10, 11]], sp)[0].outputs[0].token_ids


def test_fp32_lm_head_flag_and_env(monkeypatch):
    base = LLM(**KW)
    fp32 = LLM(fp32_lm_head=True, **KW)
    assert fp32.engine.config.fp32_lm_head and not base.engine.config.fp32_lm_head
    h = torch.randn(3, base.engine.config.model.hidden_size).to(torch.bfloat16)
    a = base.engine.runner.model.compute_logits(h)
    b = fp32.engine.runner.model.compute_logits(h, fp32=True)
    assert b.dtype == torch.float32 and a.dtype == torch.bfloat16
    assert torch.allclose(a.float(), b, atol=5e-2, rtol=5e-2)
    assert len(_greedy(fp32)) == 8
    monkeypatch.setenv("ARCTIC_FP32_LM_HEAD", "1")
    assert EngineArgs(model="llama-tiny").fp32_lm_head


def test_max_tokens_n_gives_each_sample_its_length():
    llm = LLM(**KW)
    sp = SamplingParams(temperature=0.8, seed=1, n=3, max_tokens=50, max_tokens_n=[2, 7, 4], ignore_eos=True)
    out = llm.generate([[5, 6, 7]], sp)[0]
    assert [len(c.token_ids) for c in out.outputs] == [2, 7, 4]
    assert [c.index for c in out.outputs] == [0, 1, 2]


def test_truncated_sampling_draws_fresh_noise_every_step():
    """An unseeded top-p request must not repeat one quantile step after step: on a uniform
    distribution its draws differ from row to row and from step to step."""
    from types import SimpleNamespace
    from arcticinference_b200.engine.sampler import sample_full

    def draws(request_id, seed, n_tokens, mates=0):
        sp = SamplingParams(temperature=1.0, top_p=0.95, seed=seed)
        sched, rows = [], []
        for m in range(mates):   # batch-mates come first and shift this request's row
            sched.append(SimpleNamespace(request=SimpleNamespace(
                sampling_params=SamplingParams(temperature=1.0, top_k=50), request_id="mate%d" % m,
                num_tokens=3 + m, grammar=None, spec_token_ids=[]), num_draft=0))
            rows.append([m])
        sched.append(SimpleNamespace(request=SimpleNamespace(
            sampling_params=sp, request_id=request_id, num_tokens=n_tokens, grammar=None,
            spec_token_ids=[]), num_draft=0))
        rows.append([mates])
        logits = torch.zeros(mates + 1, 1000)
        return int(sample_full(logits, sched, rows)[mates])

    unseeded = [draws("req-a", None, 10 + i) for i in range(8)]
    assert len(set(unseeded)) >= 6
    assert unseeded == [draws("req-a", None, 10 + i) for i in range(8)]      # same id, same key
    # a seeded request's token does not depend on who shares the step
    assert [draws("x", 7, 20 + i) for i in range(4)] == [draws("x", 7, 20 + i, mates=3) for i in range(4)]
    assert draws("x", 7, 20) != draws("x", 8, 20) or draws("x", 7, 21) != draws("x", 8, 21)


def test_stop_strings_cut_the_output():
    llm = LLM(**KW)
    free = llm.generate([[7, 8, 9, 10, 11]], SamplingParams(temperature=0.0, max_tokens=24,
                                                           ignore_eos=True))[0].outputs[0]
    assert len(free.text) > 8 and free.finish_reason == "length"
    stop = free.text[5:8]
    at = free.text.find(stop)
    out = llm.generate([[7, 8, 9, 10, 11]], SamplingParams(temperature=0.0, max_tokens=24,
                                                          ignore_eos=True, stop=[stop]))[0].outputs[0]
    assert out.finish_reason == "stop" and out.text == free.text[:at]
    assert len(out.token_ids) < len(free.token_ids)
    kept = llm.generate([[7, 8, 9, 10, 11]], SamplingParams(
        temperature=0.0, max_tokens=24, ignore_eos=True, stop=stop,
        include_stop_str_in_output=True))[0].outputs[0]
    assert kept.text == free.text[:at + len(stop)]
    assert not llm.engine.scheduler.has_work() and llm.engine.kv_manager.usage == 0


def test_abort_reaches_every_sample_of_a_parallel_request():
    llm = LLM(**KW)
    eng = llm.engine
    eng.add_request("par", [5, 6, 7], SamplingParams(temperature=0.8, seed=1, n=3, max_tokens=40,
                                                     ignore_eos=True))
    eng.add_request("solo", [5, 6, 7], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    for _ in range(3):
        eng.step()
    eng.abort_request("par")
    assert "par" not in eng._parents
    assert [r.request_id for r in eng.scheduler.running + list(eng.scheduler.waiting)] == ["solo"]
    done = []
    while eng.has_unfinished_requests():
        done += eng.step()
    assert [o.request_id for o in done] == ["solo"] and eng.kv_manager.usage == 0


def test_options_that_cannot_be_honoured_are_refused():
    import pytest
    for kw in (dict(pipeline_parallel_size=2, tensor_parallel_size=2),
               dict(enable_expert_parallel=True), dict(kv_cache_dtype="nvfp4")):
        with pytest.raises(NotImplementedError):
            EngineArgs(model="llama-tiny", **kw).create_engine_config()
    EngineArgs(model="llama-tiny", kv_cache_dtype="auto").create_engine_config()
    EngineArgs(model="llama-tiny", pipeline_parallel_size=2).create_engine_config()   # whole-model stages


def test_every_end_of_sequence_id_of_the_checkpoint_ends_a_request(tmp_path):
    """Instruction-tuned checkpoints list several end-of-sequence ids (config.json and
    generation_config.json): each of them ends a request, unless it asks to ignore EOS."""
    import json
    from arcticinference_b200.config import ModelConfig
    base = dict(model_type="llama", hidden_size=128, num_attention_heads=2, num_hidden_layers=1,
                head_dim=64, vocab_size=1000)
    (tmp_path / "config.json").write_text(json.dumps(dict(base, eos_token_id=[7, 9])))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 11, 9]}))
    cfg = ModelConfig.from_pretrained(str(tmp_path))
    assert cfg.eos_token_id == 7 and cfg.extra_eos_token_ids == (9, 11)
    (tmp_path / "config.json").write_text(json.dumps(dict(base, eos_token_id=5)))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    cfg = ModelConfig.from_pretrained(str(tmp_path))
    assert cfg.eos_token_id == 5 and cfg.extra_eos_token_ids == ()

    kw = dict(model="llama-tiny", device="cpu", max_model_len=128, num_gpu_blocks_override=32,
              block_size=16)
    prompt = [{"prompt_token_ids": list(range(5, 30))}]
    free = LLM(**kw).generate(prompt, SamplingParams(temperature=0, max_tokens=8, ignore_eos=True))
    toks = free[0].outputs[0].token_ids
    stop_at = next(i for i, t in enumerate(toks) if t not in toks[:i] and i >= 2)
    llm = LLM(hf_overrides={"extra_eos_token_ids": (toks[stop_at],)}, **kw)
    out = llm.generate(prompt, SamplingParams(temperature=0, max_tokens=8))[0].outputs[0]
    assert out.token_ids == toks[:stop_at + 1] and out.finish_reason == "stop"
    out = llm.generate(prompt, SamplingParams(temperature=0, max_tokens=8, ignore_eos=True))
    assert out[0].outputs[0].token_ids == toks and out[0].outputs[0].finish_reason == "length"


def test_data_parallel_replicas_are_not_one_engine():
    from arcticinference_b200.config import EngineArgs
    with pytest.raises(NotImplementedError, match="replica"):
        EngineArgs(model="llama-tiny", data_parallel_size=2).create_engine_config()
