"""The top-k / top-p selection kernel on a GPU against its PyTorch restatement and the
sort-based formulation, and sampling through the engine with a truncated distribution."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams, ops
from arcticinference_b200.engine.sampler import apply_top_k_top_p
from arcticinference_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.mark.parametrize("V", [1000, 4099, 128256])
def test_topk_topp_mask_kernel(V):
    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(8, V, generator=g) * 3.0)
    logits[4, 100:130] = logits[4].topk(5).values[-1]  # equal values across the top-k boundary
    logits[1, 300:420] = logits[1].topk(45).values[-1]
    logits[0, :40] = float("-inf")                    # tokens a grammar masked
    temp = torch.tensor([1.0, 0.7, 1.3, 0.2, 1.0, 2.0, 1.0, 0.9])
    top_k = torch.tensor([0, 50, 1, 0, 7, V + 5, 20, 0], dtype=torch.int64)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.3, 0.99, 0.0, 1.0])
    want = ref.topk_topp_mask(logits, temp, top_k, top_p)
    got = ops.topk_topp_mask(logits.to(DEV), temp.to(DEV), top_k.to(DEV), top_p.to(DEV)).cpu()
    ops.check_status()
    kept_g, kept_w = torch.isfinite(got), torch.isfinite(want)
    assert int((kept_g != kept_w).sum(-1).max()) <= 1        # the token on the boundary
    both = kept_g & kept_w
    assert torch.allclose(got[both], want[both], rtol=1e-6, atol=1e-6)
    assert kept_g[2].sum() == 1 and kept_g[6].sum() == 1 and kept_g[1].sum() == 50
    assert kept_g[7].all() and kept_g[4].sum() <= 7
    # and against sorting, on the rows that have a top-p cut
    srt = apply_top_k_top_p((logits / temp.clamp(min=1e-5).unsqueeze(1)).to(DEV), top_k.to(DEV),
                            top_p.to(DEV)).cpu()
    rows = [0, 2, 3, 5, 6]                                   # (rows 1 and 4 have ties at the k-th place)
    assert int((kept_g != torch.isfinite(srt))[rows].sum(-1).max()) <= 1
    # no argument is optional in the kernel's eyes only: off switches give the scaled logits
    plain = ops.topk_topp_mask(logits.to(DEV)).cpu()
    assert torch.equal(plain, logits)


def test_truncated_sampling_through_the_engine():
    llm = LLM(model="llama-tiny", device=DEV, num_gpu_blocks_override=128, block_size=16,
              max_model_len=512)
    prompts = [{"prompt_token_ids": list(range(5, 60))}, {"prompt_token_ids": [4, 8, 15, 16, 23]}]
    greedy = llm.generate(prompts, SamplingParams(temperature=0, max_tokens=8, ignore_eos=True))
    # top_k = 1 leaves one token per step: sampling at any temperature is greedy decoding
    one = llm.generate(prompts, SamplingParams(temperature=1.5, top_k=1, max_tokens=8,
                                               ignore_eos=True))
    for a, b in zip(greedy, one):
        assert a.outputs[0].token_ids == b.outputs[0].token_ids
    # a seeded top-p request is reproducible, and two seeds differ
    sp = lambda s: SamplingParams(temperature=1.0, top_p=0.9, top_k=40, seed=s, max_tokens=16,
                                  ignore_eos=True)
    a = llm.generate(prompts[:1], sp(1))[0].outputs[0].token_ids
    b = llm.generate(prompts[:1], sp(1))[0].outputs[0].token_ids
    c = llm.generate(prompts[:1], sp(2))[0].outputs[0].token_ids
    ops.check_status()
    assert a == b and a != c
