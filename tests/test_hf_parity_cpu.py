"""Checkpoints written by Hugging Face transformers load into the engine and give the same
next-token distribution as the transformers implementation (fp32, CPU) of the same
architecture: Llama (llama3 rope scaling, grouped-query attention), Mistral, Qwen2 (QKV bias),
Qwen3 (per-head query / key norms, head_dim * heads != hidden_size; also with YaRN scaling). Teacher-forced: the log-probability of
every prompt token given the tokens before it, so one near-tie cannot derail the comparison.
Query and key projections are scaled up so that attention is sharp and a wrong rotary
frequency, a missing norm or a wrong head mapping moves the result by far more than bf16
rounding does."""

import pytest
import torch

transformers = pytest.importorskip("transformers")

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402

COMMON = dict(hidden_size=128, num_hidden_layers=2, intermediate_size=256, vocab_size=1000,
              head_dim=64, max_position_embeddings=512, tie_word_embeddings=False,
              eos_token_id=None, bos_token_id=1)
LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}


def _make(kind: str):
    t = transformers
    if kind == "llama":
        cfg = t.LlamaConfig(num_attention_heads=4, num_key_value_heads=2, rope_theta=500000.0,
                            rope_scaling=dict(LLAMA3), rms_norm_eps=1e-5, **COMMON)
        return t.LlamaForCausalLM(cfg)
    if kind == "mistral":
        cfg = t.MistralConfig(num_attention_heads=2, num_key_value_heads=1, rope_theta=1000000.0,
                              rms_norm_eps=1e-5, sliding_window=None, **COMMON)
        return t.MistralForCausalLM(cfg)
    if kind == "qwen2-gqa3":
        # three query heads per K/V head: not a divisor of the kernels' 128-row tiles, so the
        # engine stores every K/V head three times
        cfg = t.Qwen2Config(num_attention_heads=6, num_key_value_heads=2, rope_theta=1000000.0,
                            rms_norm_eps=1e-6, use_sliding_window=False,
                            **{k: v for k, v in COMMON.items() if k != "head_dim"})
        cfg.hidden_size = 384
        return t.Qwen2ForCausalLM(cfg)
    if kind == "qwen2":
        cfg = t.Qwen2Config(num_attention_heads=4, num_key_value_heads=2, rope_theta=1000000.0,
                            rms_norm_eps=1e-6, use_sliding_window=False,
                            **{k: v for k, v in COMMON.items() if k != "head_dim"})
        cfg.hidden_size = 256          # Qwen2 has no head_dim field: hidden_size / heads = 64
        return t.Qwen2ForCausalLM(cfg)
    extra = {}
    if kind == "qwen3-yarn":          # the long-context form: prompt positions beyond the original 64
        extra = dict(rope_scaling={"rope_type": "yarn", "factor": 4.0,
                                   "original_max_position_embeddings": 64})
    cfg = t.Qwen3Config(num_attention_heads=4, num_key_value_heads=2, rope_theta=1000000.0,
                        rms_norm_eps=1e-6, use_sliding_window=False, **extra, **COMMON)
    return t.Qwen3ForCausalLM(cfg)


def _prompt_logprobs(path, ids, **kw):
    llm = LLM(model=path, max_model_len=256, device="cpu", **kw)
    out = llm.generate([{"prompt_token_ids": ids}],
                       SamplingParams(temperature=0, max_tokens=1, prompt_logprobs=0))
    return llm, out[0].prompt_logprobs[1:]


@pytest.mark.parametrize("kind", ["llama", "mistral", "qwen2", "qwen2-gqa3", "qwen3", "qwen3-yarn"])
def test_prompt_logprobs_match_transformers(kind, tmp_path):
    torch.manual_seed(0)
    m = _make(kind).float().eval()
    with torch.no_grad():
        for name, p in m.named_parameters():
            if "q_norm" in name or "k_norm" in name:
                p.copy_(1 + 0.3 * torch.randn_like(p))
            elif name.endswith("proj.bias"):
                p.copy_(0.5 * torch.randn_like(p))
            elif not kind.startswith("qwen3") and ("q_proj" in name or "k_proj" in name):
                p.mul_(6.0)          # (Qwen3's norms already make its attention sharp)
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    ids = torch.randint(2, 1000, (1, 100))
    with torch.no_grad():
        lg = m(ids).logits.log_softmax(-1)
    ref = [lg[0, i, ids[0, i + 1]].item() for i in range(99)]

    llm, got = _prompt_logprobs(str(tmp_path), ids[0].tolist())
    cfg = llm.engine.config.model
    assert cfg.rope_theta == (500000.0 if kind == "llama" else 1000000.0)
    assert cfg.qk_norm == kind.startswith("qwen3") and cfg.qkv_bias == kind.startswith("qwen2")
    if kind == "qwen2-gqa3":
        assert (cfg.num_key_value_heads, cfg.checkpoint_kv_heads, cfg.kv_head_replication) == (6, 2, 3)
        lw = llm.engine.runner.model.layers[0]
        D = 64
        assert lw.wqkv.shape[0] == (6 + 6 + 6) * D and lw.bqkv.shape[0] == 18 * D
        # the trainer-facing view keeps the checkpoint's shapes, and exporting gives them back
        from arcticinference_b200.server.weight_sync.utils import (expected_llama_tensors,
                                                                   export_llama_state)
        shapes = {t.name: tuple(t.shape) for t in expected_llama_tensors(cfg)}
        assert shapes["model.layers.0.self_attn.k_proj.weight"] == (2 * D, 384)
        assert shapes["model.layers.1.self_attn.v_proj.bias"] == (2 * D,)
        back = dict(export_llama_state(llm.engine.runner.model))
        sd = m.state_dict()
        for name in ("model.layers.0.self_attn.k_proj.weight", "model.layers.1.self_attn.v_proj.bias",
                     "model.layers.1.self_attn.q_proj.weight"):
            assert torch.equal(back[name].float(), sd[name].to(torch.bfloat16).float())
    assert (cfg.rope_scaling or {}).get("rope_type") == {"llama": "llama3",
                                                         "qwen3-yarn": "yarn"}.get(kind)
    err = max(abs(a - b) for a, b in zip(ref, got))
    assert err < 0.03, err

    # the comparison notices what it is there to notice
    wrong = {"qk_norm": False} if kind == "qwen3" else \
        {"rope_scaling": None} if kind == "qwen3-yarn" else {"rope_theta": 10000.0}
    _, off = _prompt_logprobs(str(tmp_path), ids[0].tolist(), hf_overrides=wrong)
    assert max(abs(a - b) for a, b in zip(ref, off)) > 5 * max(err, 0.01)


def test_unsupported_architectures_are_refused():
    from arcticinference_b200.config import ModelConfig
    base = dict(hidden_size=128, num_attention_heads=4, num_hidden_layers=2)
    # a windowed checkpoint is served up to its window and refused beyond it
    from arcticinference_b200.config import EngineArgs
    import dataclasses
    win = ModelConfig.from_hf_dict(dict(base, model_type="mistral", sliding_window=64, head_dim=64,
                                        num_key_value_heads=2, max_position_embeddings=32768))
    assert win.sliding_window == 64

    def engine_config(max_len):
        args = EngineArgs(model="llama-tiny", max_model_len=max_len,
                          hf_overrides={"sliding_window": 64})
        return args.create_engine_config()
    assert engine_config(64).scheduler.max_model_len == 64
    with pytest.raises(NotImplementedError, match="sliding-window"):
        engine_config(65)
    with pytest.raises(NotImplementedError, match="bias"):
        ModelConfig.from_hf_dict(dict(base, model_type="llama", attention_bias=True))
    with pytest.raises(NotImplementedError, match="model_type"):
        ModelConfig.from_hf_dict(dict(base, model_type="qwen3_moe"))
    # Qwen3 checkpoints carry a window size that is switched off
    cfg = ModelConfig.from_hf_dict(dict(base, model_type="qwen3", head_dim=64, sliding_window=4096,
                                        use_sliding_window=False, max_position_embeddings=40960))
    assert cfg.qk_norm and cfg.head_dim == 64
    from arcticinference_b200.models.llama import compute_inv_freq
    cfg.rope_scaling = {"rope_type": "longrope", "factor": 4.0}
    with pytest.raises(NotImplementedError, match="longrope"):
        compute_inv_freq(cfg, "cpu")


@pytest.mark.parametrize("pooling", ["cls", "mean"])
def test_bert_embeddings_match_transformers(pooling, tmp_path):
    from arcticinference_b200.embedding.engine import EmbeddingEngine
    torch.manual_seed(0)
    cfg = transformers.BertConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=2,
                                  intermediate_size=256, vocab_size=1000,
                                  max_position_embeddings=128, type_vocab_size=2)
    m = transformers.BertModel(cfg, add_pooling_layer=False).float().eval()
    with torch.no_grad():
        for name, p in m.named_parameters():       # norms and biases away from their 1 / 0 init
            if "LayerNorm" in name:
                p.add_(0.2 * torch.randn_like(p))
            elif "bias" in name:
                p.add_(0.1 * torch.randn_like(p))
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    eng = EmbeddingEngine(model=str(tmp_path), device="cpu", dtype=torch.float32)
    seqs = [torch.randint(5, 1000, (n,)).tolist() for n in (7, 50, 128, 1)]
    got = torch.from_numpy(eng.encode(seqs, pooling=pooling)).float()
    want = []
    with torch.no_grad():
        for s in seqs:
            h = m(torch.tensor([s])).last_hidden_state[0]
            want.append(torch.nn.functional.normalize(h[0] if pooling == "cls" else h.mean(0), dim=0))
    assert (got - torch.stack(want)).abs().max().item() < 1e-5
