"""Qwen3 on a GPU: the per-head query / key norm kernel against its fp32 PyTorch restatement,
and the engine (eager and CUDA-graph decode) against the CPU path."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams, ops
from arcticinference_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("T,Hq,Hkv,D,pad", [(1, 8, 2, 64, 0), (37, 4, 4, 128, 0), (5, 64, 8, 128, 0),
                                            (300, 3, 1, 64, 64), (9, 16, 0, 128, 8),
                                            (4099, 8, 2, 128, 0)])
def test_qk_norm_kernel(T, Hq, Hkv, D, pad):
    torch.manual_seed(T + Hq)
    width = (Hq + 2 * max(Hkv, 1)) * D
    buf = _rand(T, width + pad, scale=3.0)
    qkv = buf[:, :width]                       # row stride wider than the row when pad > 0
    wq, wk = _rand(D, scale=0.3) + 1.0, _rand(D, scale=0.3) + 1.0
    want = ref.qk_norm(qkv.float().clone(), wq, wk, Hq, Hkv, D, 1e-6)
    before = buf.clone()
    ops.qk_norm(qkv, wq, wk, Hq, Hkv, D, 1e-6)
    ops.check_status()
    n = (Hq + Hkv) * D
    err = (qkv[:, :n].float() - want[:, :n]).abs()
    assert float(err.max()) < 0.03 * max(1.0, float(want[:, :n].abs().max())), float(err.max())
    # the value heads and the padding are untouched
    assert torch.equal(buf[:, n:], before[:, n:])


def _copy_weights(src, dst):
    for (n1, t1), (n2, t2) in zip(src.named_tensors(), dst.named_tensors()):
        assert n1 == n2
        t2.copy_(t1.to(t2.device))


def _first_logits(llm, prompts):
    eng = llm.engine
    for p in prompts:
        eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=4, ignore_eos=True))
    out = eng.scheduler.schedule()
    batch, rows = eng.runner.prepare(out)
    with torch.inference_mode():
        h = eng.runner.model.forward(batch, eng.runner.kv)
        return eng.runner.model.compute_logits(h).float().cpu()


def test_qwen3_forward_matches_the_cpu_path():
    kw = dict(model="qwen3-tiny", num_gpu_blocks_override=128, block_size=16, max_model_len=1024)
    gpu, cpu = LLM(device="cuda:0", **kw), LLM(device="cpu", **kw)
    names = [n for n, _ in gpu.engine.runner.model.named_tensors()]
    assert "layers.0.q_norm" in names and "layers.1.k_norm" in names
    _copy_weights(gpu.engine.runner.model, cpu.engine.runner.model)
    prompts = [list(range(3, 150)), [9, 8, 7, 6], list(range(200, 260))]
    a, b = _first_logits(gpu, prompts), _first_logits(cpu, prompts)
    ops.check_status()
    err = (a - b).abs().max().item()
    assert err < 0.08 * max(1.0, b.abs().max().item()), err


def test_qwen3_cuda_graph_decode_matches_eager():
    sp = SamplingParams(temperature=0, max_tokens=12, ignore_eos=True)
    prompts = [{"prompt_token_ids": list(range(5, 5 + n))} for n in (40, 7, 300, 65, 130)]
    kw = dict(model="qwen3-tiny", device="cuda:0", num_gpu_blocks_override=256, block_size=16,
              max_model_len=1024)
    a = LLM(enforce_eager=True, **kw).generate(prompts, sp)
    graphed = LLM(enforce_eager=False, **kw)
    b = graphed.generate(prompts, sp)
    ops.check_status()
    assert graphed.engine.runner.graph_replays > 0
    for x, y in zip(a, b):
        assert x.outputs[0].token_ids == y.outputs[0].token_ids
