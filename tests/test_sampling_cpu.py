"""Top-k / top-p truncation by selection instead of sorting: the PyTorch restatement against
the sort-based formulation, and the kernel's search (bit-wise selection of the k-th largest
key, bisection on the key for the top-p cut) replayed with numpy against the restatement."""

import numpy as np
import pytest
import torch

from arcticinference_b200 import ops
from arcticinference_b200.engine.sampler import apply_top_k_top_p
from arcticinference_b200.ops import reference as ref


def _keys(y: np.ndarray) -> np.ndarray:
    u = y.astype(np.float32).view(np.uint32)
    return np.where(u & 0x80000000, ~u, u | 0x80000000).astype(np.uint64)


def _replay_kernel_row(x, temp, k, p):
    """The search of csrc/sampling.cu for one row, pass by pass."""
    V = x.size
    inv_t = np.float32(1.0) / max(np.float32(temp), np.float32(1e-5))
    y = (x.astype(np.float32) * inv_t).astype(np.float32)
    key = _keys(y)
    if k <= 0 or k > V:
        k = V
    k_key, tie_end = 0, 0xffffffff
    idx = np.arange(V)
    if k < V:
        for bit in range(31, -1, -1):
            cand = k_key | (1 << bit)
            if int((key >= cand).sum()) >= k:
                k_key = cand
        above, equal = int((key > k_key).sum()), int((key == k_key).sum())
        need = k - above
        assert 1 <= need <= equal
        if equal > need:
            tie_end = 0
            for bit in range(31, -1, -1):
                cand = tie_end | (1 << bit)
                if int(((idx < cand) & (key == k_key)).sum()) <= need:
                    tie_end = cand
    in_k = (key > k_key) | ((key == k_key) & (idx < tie_end))
    keep_key = k_key
    if p < 1.0:
        m = y.max()
        w = np.exp((y - m).astype(np.float32)).astype(np.float32)
        z = w[in_k].sum(dtype=np.float32)
        target = np.float32(p) * z
        lo, hi = k_key, int(_keys(np.array([m]))[0])
        steps = 0
        while lo < hi:
            mid = lo + ((hi - lo) >> 1)
            s = w[key > mid].sum(dtype=np.float32)
            if s <= target:
                hi = mid
            else:
                lo = mid + 1
            steps += 1
        assert steps <= 32
        keep_key = hi
    return np.where((key >= keep_key) & in_k, y, -np.inf).astype(np.float32)


def _cases(B, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(B, V, generator=g) * 3.0
    temp = torch.tensor([1.0, 0.7, 1.3, 0.2, 1.0, 2.0, 1.0, 0.9][:B])
    top_k = torch.tensor([0, 50, 1, 0, 7, V + 5, 20, 0][:B], dtype=torch.int64)
    top_p = torch.tensor([0.9, 1.0, 0.5, 0.95, 0.3, 0.99, 0.0, 1.0][:B])
    return logits, temp, top_k, top_p


@pytest.mark.parametrize("V", [1000, 4099])
def test_selection_matches_the_sort_based_formulation(V):
    logits, temp, top_k, top_p = _cases(8, V, seed=V)
    got = ops.topk_topp_mask(logits, temp, top_k, top_p)
    want = apply_top_k_top_p(logits / temp.clamp(min=1e-5).unsqueeze(1), top_k, top_p)
    kept_g, kept_w = torch.isfinite(got), torch.isfinite(want)
    # continuous random logits: no ties; the two differ at most in the token that sits on the
    # probability boundary (different summation orders)
    # (with top_p = 1 the sort-based form drops tail tokens once its running sum rounds above
    # 1; the selection treats top_p >= 1 as off)
    cut = top_p < 1.0
    assert int((kept_g != kept_w)[cut].sum(-1).max()) <= 1
    both = kept_g & kept_w
    assert torch.allclose(got[both], want[both], rtol=1e-6, atol=1e-6)
    assert kept_g[2].sum() == 1 and kept_g[6].sum() == 1          # top_k = 1; top_p = 0
    assert kept_g[1].sum() == 50 and kept_g[7].all()              # top_k only; nothing


def test_equal_logits():
    x = torch.tensor([[1.0, 2.0, 1.0, 1.0, 0.0, -1.0]])
    one = torch.ones(1)
    # ties for the k-th place go to the lowest token ids: exactly k survive
    for k, kept in ((1, [1]), (2, [0, 1]), (3, [0, 1, 2]), (4, [0, 1, 2, 3]), (5, [0, 1, 2, 3, 4])):
        out = ops.topk_topp_mask(x, one, torch.tensor([k]), one)
        assert torch.isfinite(out)[0].nonzero().flatten().tolist() == kept
    flat = torch.zeros(1, 9)
    assert torch.isfinite(ops.topk_topp_mask(flat, one, torch.tensor([1]), one))[0].tolist() == \
        [True] + [False] * 8
    # mass above the 1.0 tokens is e^2 / Z = 0.42: with top_p = 0.4 they all go, with 0.45 all stay
    for p, n in ((0.4, 1), (0.45, 4)):
        out = ops.topk_topp_mask(x, one, None, torch.tensor([p]))
        assert int(torch.isfinite(out).sum()) == n


def test_kernel_search_replayed_on_the_host():
    logits, temp, top_k, top_p = _cases(8, 2500, seed=3)
    logits[4, 100:130] = logits[4].topk(5).values[-1]  # equal values across the top-k boundary
    logits[1, 300:420] = logits[1].topk(45).values[-1]
    logits[0, :40] = float("-inf")                    # tokens a grammar masked
    want = ref.topk_topp_mask(logits, temp, top_k, top_p).numpy()
    for b in range(8):
        got = _replay_kernel_row(logits[b].numpy(), float(temp[b]), int(top_k[b]), float(top_p[b]))
        diff = np.isfinite(got) != np.isfinite(want[b])
        assert diff.sum() <= 1, (b, diff.sum())
        same = np.isfinite(got) & np.isfinite(want[b])
        np.testing.assert_allclose(got[same], want[b][same], rtol=1e-6)


KW = dict(model="llama-tiny", device="cpu", num_gpu_blocks_override=64, block_size=16, max_model_len=256)


def _gen(llm, **sp):
    from arcticinference_b200 import SamplingParams
    out = llm.generate([{"prompt_token_ids": list(range(5, 40))}],
                       SamplingParams(max_tokens=24, ignore_eos=True, **sp))
    return out[0].outputs[0].token_ids


def test_penalties_bias_and_min_p_through_the_engine():
    from arcticinference_b200 import LLM
    llm = LLM(**KW)
    plain = _gen(llm, temperature=0)
    assert len(set(plain)) < len(plain)                     # a tiny random model repeats itself
    # a large frequency penalty: no token twice
    assert len(set(_gen(llm, temperature=0, frequency_penalty=100.0))) == 24
    assert len(set(_gen(llm, temperature=0, presence_penalty=100.0))) == 24
    # repetition penalty also covers the prompt: nothing from the prompt, nothing twice
    rep = _gen(llm, temperature=0, repetition_penalty=1e4)
    assert len(set(rep)) == 24 and not set(rep) & set(range(5, 40))
    # neutral values change nothing
    assert _gen(llm, temperature=0, repetition_penalty=1.0, presence_penalty=0.0, min_p=0.0) == plain
    # a bias picks the token; a negative one bans the model's favourites
    assert _gen(llm, temperature=0, logit_bias={"77": 100.0}) == [77] * 24
    banned = _gen(llm, temperature=0, logit_bias={t: -100.0 for t in set(plain)})
    assert not set(banned) & set(plain)
    # min_p = 1 leaves only the most likely token: sampling is greedy decoding
    assert _gen(llm, temperature=1.0, min_p=1.0, seed=3) == plain
    # and a small min_p still samples (differs from greedy with this seed)
    assert _gen(llm, temperature=1.5, min_p=0.001, seed=3) != plain


def test_penalty_arithmetic():
    from types import SimpleNamespace as NS
    from arcticinference_b200 import SamplingParams
    from arcticinference_b200.engine.sampler import apply_penalties
    lf = torch.tensor([[2.0, -2.0, 1.0, 0.5, 0.0, 3.0]])
    sp = SamplingParams(repetition_penalty=2.0, presence_penalty=0.5, frequency_penalty=0.25,
                        logit_bias={5: -1.0, 99: 7.0})
    req = NS(sampling_params=sp, prompt_token_ids=[0, 1], output_token_ids=[2, 2, 3], spec_token_ids=[])
    out = apply_penalties(lf, [NS(request=req, num_draft=0)], [[0]])
    # prompt tokens 0, 1 and generated 2, 3: repetition (positive halved, negative doubled);
    # generated 2 (twice) and 3 (once): presence + frequency; token 5: bias
    want = [1.0, -4.0, 0.5 - 0.5 - 0.5, 0.25 - 0.5 - 0.25, 0.0, 2.0]
    assert torch.allclose(out[0], torch.tensor(want)) and torch.equal(lf[0, :2], torch.tensor([2.0, -2.0]))
