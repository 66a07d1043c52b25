"""Engine options that have no test elsewhere: the fp32 LM head (flag and environment
switch) and per-sample forced lengths for rollout replay."""

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
