"""Speculative decoding must never change greedy outputs; suffix drafts must get accepted on
repetitive text; batch-size caps and draft bookkeeping."""

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import SpeculativeConfig
from arcticinference_b200.ops import spec_ops

KW = dict(model="llama-tiny", device="cpu", num_gpu_blocks_override=128, block_size=16,
          max_model_len=512)
PROMPTS = [{"prompt_token_ids": [5, 6, 7, 8, 9, 10] * 8}, {"prompt_token_ids": list(range(40, 75))},
           {"prompt_token_ids": [3, 3, 3, 4, 4, 4] * 5}]
SP = SamplingParams(temperature=0, max_tokens=24, ignore_eos=True)


def _tokens(outs):
    return [o.outputs[0].token_ids for o in outs]


@pytest.fixture(scope="module")
def baseline():
    return _tokens(LLM(**KW).generate(PROMPTS, SP))


@pytest.mark.parametrize("spec", [
    {"method": "suffix"},
    {"method": "arctic", "model": "random", "num_speculative_tokens": 3},
    {"method": "mlp_speculator", "model": "random", "num_speculative_tokens": 2},
    {"method": "arctic", "model": "random", "num_speculative_tokens": 3,
     "enable_suffix_decoding": True},
])
def test_speculation_preserves_greedy_output(spec, baseline):
    llm = LLM(speculative_config=spec, **KW)
    outs = llm.generate(PROMPTS, SP)
    assert _tokens(outs) == baseline
    st = llm.engine.stats
    assert st["draft_tokens"] > 0
    if spec.get("method") == "suffix" or spec.get("enable_suffix_decoding"):
        # greedy decoding of a tiny random model falls into loops that the trees pick up
        assert st["accepted_tokens"] > 0
        assert st["steps"] < 3 + 24 * 1  # fewer engine steps than one per token


def test_batch_size_caps():
    c = SpeculativeConfig(method="suffix", disable_by_batch_size=2, hard_disable_by_batch_size=4)
    assert c.effective_draft_limit(1) == 1
    assert c.effective_draft_limit(2) == 2
    assert c.effective_draft_limit(3) == 2      # soft cap: first N requests only
    assert c.effective_draft_limit(4) == 0      # hard cap: nobody drafts
    d = SpeculativeConfig(method="suffix")
    assert d.disable_by_batch_size == 64 and d.num_speculative_tokens == 16
    h = SpeculativeConfig(method="arctic", model="x", enable_suffix_decoding=True)
    assert h.suffix_speculative_tokens == h.suffix_cache_max_depth == 64
    with pytest.raises(ValueError):
        SpeculativeConfig(method="arctic")
    with pytest.raises(ValueError):
        SpeculativeConfig(method="eagle")


def test_hard_cap_disables_drafting_in_engine(baseline):
    llm = LLM(speculative_config={"method": "suffix", "hard_disable_by_batch_size": 2}, **KW)
    outs = llm.generate(PROMPTS, SP)
    assert _tokens(outs) == baseline
    # three requests decode together, so no step may carry draft tokens
    assert llm.engine.stats["draft_tokens"] == 0


def test_verify_greedy_reference():
    #            req0: token + 3 drafts     req1: token only   req2: token + 2 drafts
    input_ids = torch.tensor([10, 11, 12, 13, 20, 30, 31, 32])
    target = torch.tensor([11, 12, 99, 14, 21, 31, 32, 33])
    row_start = torch.tensor([0, 4, 5], dtype=torch.int32)
    num_draft = torch.tensor([3, 0, 2], dtype=torch.int32)
    acc, nxt, sel, out = spec_ops.verify_greedy(input_ids, target, row_start, num_draft, 3)
    assert acc.tolist() == [2, 0, 2]
    assert nxt.tolist() == [99, 21, 33]
    assert sel.tolist() == [2, 4, 7]
    assert out.tolist() == [[11, 12, 99, -1], [21, -1, -1, -1], [31, 32, 33, -1]]


def test_fp8_speculator_keeps_outputs(baseline):
    llm = LLM(speculative_config={"method": "arctic", "model": "random", "num_speculative_tokens": 3,
                                  "quantization": "fp8"}, **KW)
    from arcticinference_b200.models.quant import Fp8Weight
    assert any(isinstance(t, Fp8Weight) for t in llm.engine.runner.proposer.w.values())
    assert _tokens(llm.generate(PROMPTS, SP)) == baseline
    llm.sleep(2)
    llm.wake_up()
    assert _tokens(llm.generate(PROMPTS, SP)) == baseline


def test_acceptance_histogram_by_position():
    """Drafts vary in width; the engine counts, per draft position, how often it was drafted
    and how often accepted (accepted counts never exceed drafted counts and never grow with
    the position)."""
    from arcticinference_b200 import LLM, SamplingParams
    llm = LLM(model="llama-tiny", device="cpu", max_model_len=256, num_gpu_blocks_override=64,
              speculative_config={"method": "suffix"})
    prompts = [{"prompt_token_ids": [5, 6, 7, 8] * 12}, {"prompt_token_ids": list(range(9, 60))}]
    llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40, ignore_eos=True))
    st = llm.engine.get_stats()
    drafted, accepted = st["drafted_per_position"], st["accepted_per_position"]
    assert drafted and sum(drafted) == st["draft_tokens"]
    assert sum(accepted) == st["accepted_tokens"]
    assert all(a <= d for a, d in zip(accepted, drafted))
    assert all(x >= y for x, y in zip(accepted, accepted[1:]))
    assert st["tp_steps"] == st["steps"] and st["sp_steps"] == 0


@pytest.mark.parametrize("fmt", ["bin", "safetensors"])
def test_speculator_checkpoint_round_trip(tmp_path, fmt):
    """A speculator directory holds ``config.json`` plus safetensors files or, in older
    releases, ``pytorch_model.bin`` (the reference reads both:
    arctic_inference/server/weight_sync/utils.py:437-461)."""
    import dataclasses
    import json
    import torch
    from arcticinference_b200.models.speculator import SpeculatorConfig, build_speculator
    from arcticinference_b200.utils.safetensors_io import write_safetensors
    cfg = SpeculatorConfig(n_predict=3, vocab_size=64, emb_dim=32, inner_dim=32, proj_dim=32,
                           input_hidden_dim=32, method="sum_lstm")
    src = build_speculator(cfg, device="cpu", seed=3)
    d = dataclasses.asdict(cfg)
    d["architectures"] = [d.pop("architecture")]
    (tmp_path / "config.json").write_text(json.dumps(d))
    state = {"speculator." + k: v.clone() for k, v in src.w.items()}
    if fmt == "bin":
        torch.save(state, tmp_path / "pytorch_model.bin")
    else:
        write_safetensors(str(tmp_path / "model.safetensors"), state)
    got = build_speculator(str(tmp_path), device="cpu")
    h = torch.randn(5, 32, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    tok = torch.arange(5, dtype=torch.int64)
    assert torch.equal(src.propose(h, tok, 3), got.propose(h, tok, 3))


@pytest.mark.parametrize("model", ["qwen3-tiny", "qwen2-tiny"])
def test_speculation_preserves_output_on_the_qwen_paths(model):
    """Verification rows pass through the per-head norms / the QKV bias like any other row."""
    kw = dict(KW, model=model)
    want = _tokens(LLM(**kw).generate(PROMPTS, SP))
    llm = LLM(speculative_config={"method": "arctic", "model": "random", "num_speculative_tokens": 3,
                                  "enable_suffix_decoding": True}, **kw)
    assert _tokens(llm.generate(PROMPTS, SP)) == want
    assert llm.engine.stats["draft_tokens"] > 0 and llm.engine.stats["accepted_tokens"] > 0
