"""Qwen2 on a GPU: the QKV bias rides in the GEMM epilogue; first-step logits and CUDA-graph
decode against the CPU path."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams, ops

pytestmark = pytest.mark.gpu


def test_qwen2_forward_and_graphed_decode_match_the_cpu_path():
    kw = dict(model="qwen2-tiny", num_gpu_blocks_override=128, block_size=16, max_model_len=1024)
    gpu, cpu = LLM(device="cuda:0", **kw), LLM(device="cpu", **kw)
    for (n1, t1), (n2, t2) in zip(gpu.engine.runner.model.named_tensors(),
                                  cpu.engine.runner.model.named_tensors()):
        assert n1 == n2
        t2.copy_(t1.to(t2.device))
    assert any(n.endswith("bqkv") for n, _ in gpu.engine.runner.model.named_tensors())
    prompts = [list(range(3, 150)), [9, 8, 7, 6], list(range(200, 260))]
    logits = []
    for llm in (gpu, cpu):
        eng = llm.engine
        for p in prompts:
            eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=6, ignore_eos=True))
        out = eng.scheduler.schedule()
        batch, _ = eng.runner.prepare(out)
        with torch.inference_mode():
            h = eng.runner.model.forward(batch, eng.runner.kv)
            logits.append(eng.runner.model.compute_logits(h).float().cpu())
    ops.check_status()
    err = (logits[0] - logits[1]).abs().max().item()
    assert err < 0.08 * max(1.0, logits[1].abs().max().item()), err
    # decode (token-major GEMMs, CUDA graphs) gives the same first tokens as the CPU path
    sp = SamplingParams(temperature=0, max_tokens=6, ignore_eos=True)
    fresh = dict(kw, num_gpu_blocks_override=256)
    a = LLM(device="cuda:0", **fresh)
    b = LLM(device="cpu", **fresh)
    for (_, t1), (_, t2) in zip(a.engine.runner.model.named_tensors(),
                                b.engine.runner.model.named_tensors()):
        t2.copy_(t1.to(t2.device))
    ps = [{"prompt_token_ids": p} for p in prompts]
    ga, gb = a.generate(ps, sp), b.generate(ps, sp)
    ops.check_status()
    assert a.engine.runner.graph_replays > 0
    for x, y in zip(ga, gb):
        assert x.outputs[0].token_ids[0] == y.outputs[0].token_ids[0]
