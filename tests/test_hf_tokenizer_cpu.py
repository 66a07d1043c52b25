"""A model directory with a Hugging Face tokenizer: text prompts, the chat template (whose
tokenised form is a ``BatchEncoding`` in transformers 5 and a list before), detokenised
output, and the tokenizer's EOS, through ``LLM.chat`` and the OpenAI chat endpoint."""

import json
import os

import pytest
import torch

tokenizers = pytest.importorskip("tokenizers")
transformers = pytest.importorskip("transformers")

from arcticinference_b200 import LLM, SamplingParams  # noqa: E402
from arcticinference_b200.config import PRESETS  # noqa: E402
from arcticinference_b200.models.loader import random_llama_state  # noqa: E402
from arcticinference_b200.utils.safetensors_io import write_safetensors  # noqa: E402
from arcticinference_b200.utils.tokenizer import chat_token_ids  # noqa: E402

WORDS = ("hello world how are you today write an essay about the importance of higher "
         "education ! ? .").split()
TEMPLATE = ("{% for m in messages %}{{ '<|' + m['role'] + '|> ' + m['content'] + ' <|eot|> ' }}"
            "{% endfor %}{% if add_generation_prompt %}{{ '<|assistant|> ' }}{% endif %}")


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("hf_model"))
    vocab = {"<pad>": 0, "<s>": 1, "</s>": 2, "<unk>": 3, "<|user|>": 4, "<|assistant|>": 5,
             "<|eot|>": 6}
    vocab.update({w: 7 + i for i, w in enumerate(WORDS)})
    vocab.update({"w%d" % i: i for i in range(len(vocab), 1024)})   # every model output decodes
    tk = tokenizers.Tokenizer(tokenizers.models.WordLevel(vocab, unk_token="<unk>"))
    tk.pre_tokenizer = tokenizers.pre_tokenizers.WhitespaceSplit()
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tk, bos_token="<s>",
                                                eos_token="</s>", pad_token="<pad>",
                                                unk_token="<unk>")
    fast.chat_template = TEMPLATE
    fast.save_pretrained(d)
    cfg = PRESETS["llama-tiny"]
    state = dict(random_llama_state(cfg, seed=1, std=0.05, device="cpu", dtype=torch.bfloat16))
    write_safetensors(os.path.join(d, "model.safetensors"), state)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(dict(architectures=["LlamaForCausalLM"], model_type="llama",
                       hidden_size=cfg.hidden_size, num_hidden_layers=cfg.num_hidden_layers,
                       num_attention_heads=cfg.num_attention_heads, head_dim=cfg.head_dim,
                       num_key_value_heads=cfg.num_key_value_heads,
                       intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size,
                       rope_theta=cfg.rope_theta, max_position_embeddings=512,
                       eos_token_id=2), f)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [2, 6]}, f)                 # </s> and the end-of-turn token
    return d


def test_chat_through_a_hugging_face_tokenizer(model_dir):
    llm = LLM(model=model_dir, device="cpu", max_model_len=128, num_gpu_blocks_override=32,
              block_size=16)
    tok = llm.get_tokenizer()
    assert type(tok).__name__ != "ByteTokenizer"
    conv = [{"role": "user", "content": "hello world how are you today ?"}]
    ids = chat_token_ids(tok, conv)
    assert ids == [4, 7, 8, 9, 10, 11, 12, 7 + WORDS.index("?"), 6, 5]
    assert llm.engine.config.model.extra_eos_token_ids == (6,)
    sp = SamplingParams(temperature=0, max_tokens=12)
    out = llm.chat(conv, sp)[0]
    assert out.prompt_token_ids == ids
    same = llm.generate([{"prompt_token_ids": ids}], sp)[0]
    assert out.outputs[0].token_ids == same.outputs[0].token_ids
    # the text is the detokenised output, and a text prompt goes through the same tokenizer
    assert out.outputs[0].text == tok.decode(out.outputs[0].token_ids, skip_special_tokens=True)
    txt = llm.generate(["hello world"], sp)[0]
    assert txt.prompt_token_ids == tok.encode("hello world")
    # a request that meets </s> or <|eot|> stops there
    free = llm.generate([{"prompt_token_ids": ids}],
                        SamplingParams(temperature=0, max_tokens=40, ignore_eos=True))[0]
    toks = free.outputs[0].token_ids
    stops = [i for i, t in enumerate(toks) if t in (2, 6)]
    full = llm.generate([{"prompt_token_ids": ids}], SamplingParams(temperature=0, max_tokens=40))[0]
    if stops:
        assert full.outputs[0].token_ids == toks[:stops[0] + 1]
        assert full.outputs[0].finish_reason == "stop"
    else:
        assert full.outputs[0].token_ids == toks


def test_openai_chat_endpoint_with_a_hugging_face_tokenizer(model_dir):
    from fastapi.testclient import TestClient
    from arcticinference_b200.config import EngineArgs
    from arcticinference_b200.engine.async_llm import AsyncLLM
    from arcticinference_b200.entrypoints.openai_server import build_app
    llm = AsyncLLM.from_engine_args(EngineArgs(model=model_dir, max_model_len=128, block_size=16,
                                               num_gpu_blocks_override=32), device="cpu").start()
    try:
        with TestClient(build_app(llm, "m")) as client:
            r = client.post("/v1/chat/completions", json={
                "model": "m", "max_tokens": 6, "temperature": 0,
                "messages": [{"role": "user", "content": "write an essay about education"}]})
            assert r.status_code == 200, r.text
            body = r.json()
            assert body["usage"]["prompt_tokens"] == 1 + 5 + 1 + 1
            assert isinstance(body["choices"][0]["message"]["content"], str)
    finally:
        llm.shutdown()


def test_streamed_chat_deltas_add_up_to_the_full_text(model_dir):
    from fastapi.testclient import TestClient
    from arcticinference_b200.config import EngineArgs
    from arcticinference_b200.engine.async_llm import AsyncLLM
    from arcticinference_b200.entrypoints.openai_server import build_app
    llm = AsyncLLM.from_engine_args(EngineArgs(model=model_dir, max_model_len=128, block_size=16,
                                               num_gpu_blocks_override=32), device="cpu").start()
    body = {"model": "m", "max_tokens": 10, "temperature": 0, "ignore_eos": True,
            "messages": [{"role": "user", "content": "how are you today ?"}]}
    try:
        with TestClient(build_app(llm, "m")) as client:
            whole = client.post("/v1/chat/completions", json=body).json()
            text = whole["choices"][0]["message"]["content"]
            parts = []
            with client.stream("POST", "/v1/chat/completions", json=dict(body, stream=True)) as r:
                for line in r.iter_lines():
                    if line.startswith("data: {"):
                        d = json.loads(line[6:])
                        for c in d.get("choices", []):
                            parts.append(c.get("delta", {}).get("content") or "")
            assert "".join(parts) == text and len([p for p in parts if p]) > 1
    finally:
        llm.shutdown()


def test_continue_final_message_leaves_the_last_turn_open():
    from arcticinference_b200.utils.tokenizer import ByteTokenizer
    tok = ByteTokenizer(1024)
    msgs = [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "The answer is"}]
    closed = chat_token_ids(tok, msgs, True)
    opened = chat_token_ids(tok, msgs, False, continue_final_message=True)
    assert tok.decode(opened).endswith("The answer is") and len(opened) < len(closed)
