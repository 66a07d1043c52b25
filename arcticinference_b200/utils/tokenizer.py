"""Tokenizer glue: a Hugging Face tokenizer when a model directory provides one,
otherwise a byte-level stand-in so that synthetic (random-weight) presets can be
driven with text prompts."""

from __future__ import annotations

import os
from typing import Optional


class ByteTokenizer:
    """UTF-8 bytes shifted past a few special ids; round-trips any string."""

    def __init__(self, vocab_size: int = 1024):
        self.vocab_size = vocab_size
        self.bos_token_id = 1
        self.eos_token_id = 2
        self.pad_token_id = 0
        self._offset = 3

    def encode(self, text: str, add_special_tokens: bool = True) -> list[int]:
        ids = [b + self._offset for b in text.encode("utf-8")]
        ids = [i % self.vocab_size for i in ids]
        return ([self.bos_token_id] if add_special_tokens else []) + ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        bs = bytes((i - self._offset) % 256 for i in ids
                   if not (skip_special_tokens and i < self._offset))
        return bs.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True,
                            continue_final_message=False, **kw):
        text = "".join("<|%s|>\n%s\n" % (m["role"], m["content"]) for m in messages)
        if continue_final_message:
            text = text[:-1]          # the last turn stays open
        elif add_generation_prompt:
            text += "<|assistant|>\n"
        return self.encode(text) if tokenize else text


def chat_token_ids(tokenizer, messages, add_generation_prompt: bool = True, **kw) -> list:
    """Token ids of a conversation under the tokenizer's chat template. Hugging Face
    tokenizers return a plain list (transformers 4) or a ``BatchEncoding`` with ``input_ids``
    (transformers 5, which is a ``UserDict``, not a ``dict``); both are accepted."""
    out = tokenizer.apply_chat_template(messages, tokenize=True,
                                        add_generation_prompt=add_generation_prompt, **kw)
    if hasattr(out, "keys") and "input_ids" in out:
        out = out["input_ids"]
    if len(out) and isinstance(out[0], (list, tuple)):      # a batch of one
        out = out[0]
    return [int(t) for t in out]


def get_tokenizer(name_or_path: Optional[str], vocab_size: int = 1024):
    if name_or_path and os.path.isdir(name_or_path):
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(name_or_path)
        except Exception:
            pass
    return ByteTokenizer(vocab_size)
