"""BERT-family encoder for the embedding service.

The reference serves embeddings by wrapping a vLLM pooling model
(arctic_inference/embedding/replica.py:83-128); here the encoder is part of the framework and
runs on the same kernels as the decoder stack:

* one fused kernel sums word + position + token-type rows and layer-normalises them;
* each layer is four tensor-core GEMMs whose epilogues carry the bias, the GELU and the
  residual add (QKV, attention output + residual, FFN-up + GELU, FFN-down + residual), one
  bidirectional varlen attention launch over the packed batch (no padding tokens are
  computed) and two LayerNorm launches;
* pooling (CLS / mean / last) and L2 normalisation are one kernel that writes fp32.

Sequences are packed back to back: ``input_ids`` [T], ``positions`` [T] and the sequence
lengths. Weights use Hugging Face ``BertModel`` names (with or without a ``bert.`` prefix);
Q, K and V are fused into one [3H, H] matrix at load time.
"""

from __future__ import annotations

import re
from typing import Iterable, Iterator, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..config import ModelConfig

_LAYER_RE = re.compile(r"^encoder\.layer\.(\d+)\.(.+)$")


class BertLayerWeights:
    __slots__ = ("wqkv", "bqkv", "wo", "bo", "ln1_g", "ln1_b", "wi", "bi", "wd", "bd", "ln2_g",
                 "ln2_b")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


def random_bert_state(cfg: ModelConfig, seed: int, std: float, device, dtype) -> Iterator:
    """(name, tensor) pairs of a random checkpoint in Hugging Face naming."""
    gen = torch.Generator(device=device)
    H, I = cfg.hidden_size, cfg.intermediate_size

    def rnd(tag, *shape, s=std):
        gen.manual_seed(seed * 1000003 + tag)
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * s).to(dtype)

    ones = lambda n: torch.ones(n, device=device, dtype=dtype)
    yield "embeddings.word_embeddings.weight", rnd(1, cfg.vocab_size, H)
    yield "embeddings.position_embeddings.weight", rnd(2, cfg.max_position_embeddings, H)
    yield "embeddings.token_type_embeddings.weight", rnd(3, cfg.type_vocab_size, H)
    yield "embeddings.LayerNorm.weight", ones(H)
    yield "embeddings.LayerNorm.bias", rnd(4, H)
    for l in range(cfg.num_hidden_layers):
        p = "encoder.layer.%d." % l
        b = 100 + 20 * l
        for j, nm in enumerate(("query", "key", "value")):
            yield p + "attention.self.%s.weight" % nm, rnd(b + j, H, H)
            yield p + "attention.self.%s.bias" % nm, rnd(b + 3 + j, H)
        yield p + "attention.output.dense.weight", rnd(b + 6, H, H)
        yield p + "attention.output.dense.bias", rnd(b + 7, H)
        yield p + "attention.output.LayerNorm.weight", ones(H)
        yield p + "attention.output.LayerNorm.bias", rnd(b + 8, H)
        yield p + "intermediate.dense.weight", rnd(b + 9, I, H)
        yield p + "intermediate.dense.bias", rnd(b + 10, I)
        yield p + "output.dense.weight", rnd(b + 11, H, I)
        yield p + "output.dense.bias", rnd(b + 12, H)
        yield p + "output.LayerNorm.weight", ones(H)
        yield p + "output.LayerNorm.bias", rnd(b + 13, H)


class BertEncoder:
    def __init__(self, cfg: ModelConfig, device="cuda", dtype=torch.bfloat16):
        if cfg.hidden_size != cfg.num_attention_heads * cfg.head_dim:
            raise ValueError("hidden_size must equal num_attention_heads * head_dim")
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.word = self.pos = self.type = self.emb_g = self.emb_b = None
        self.layers = [BertLayerWeights() for _ in range(cfg.num_hidden_layers)]

    # ------------------------------------------------------------------ weights
    def load_state(self, state: Iterable) -> None:
        H = self.cfg.hidden_size
        qkv: dict = {}
        put = lambda t: t.to(device=self.device, dtype=self.dtype).contiguous()
        for name, t in state:
            if name.startswith("bert."):
                name = name[5:]
            if name == "embeddings.word_embeddings.weight":
                self.word = put(t)
            elif name == "embeddings.position_embeddings.weight":
                self.pos = put(t)
            elif name == "embeddings.token_type_embeddings.weight":
                self.type = put(t)
            elif name == "embeddings.LayerNorm.weight":
                self.emb_g = put(t)
            elif name == "embeddings.LayerNorm.bias":
                self.emb_b = put(t)
            else:
                m = _LAYER_RE.match(name)
                if not m:
                    continue        # pooler, position_ids buffers, heads of other tasks
                l, rest = int(m.group(1)), m.group(2)
                if l >= len(self.layers):
                    continue
                lw = self.layers[l]
                simple = {
                    "attention.output.dense.weight": "wo", "attention.output.dense.bias": "bo",
                    "attention.output.LayerNorm.weight": "ln1_g",
                    "attention.output.LayerNorm.bias": "ln1_b",
                    "intermediate.dense.weight": "wi", "intermediate.dense.bias": "bi",
                    "output.dense.weight": "wd", "output.dense.bias": "bd",
                    "output.LayerNorm.weight": "ln2_g", "output.LayerNorm.bias": "ln2_b",
                }
                if rest in simple:
                    setattr(lw, simple[rest], put(t))
                elif rest.startswith("attention.self."):
                    _, _, which, kind = rest.split(".")
                    qkv.setdefault((l, kind), {})[which] = t
        for (l, kind), parts in qkv.items():
            fused = torch.cat([parts["query"], parts["key"], parts["value"]], 0)
            setattr(self.layers[l], "wqkv" if kind == "weight" else "bqkv", put(fused))
        missing = [n for n in ("word", "pos", "type", "emb_g", "emb_b") if getattr(self, n) is None]
        for l, lw in enumerate(self.layers):
            missing += ["layer %d %s" % (l, s) for s in lw.__slots__ if getattr(lw, s) is None]
        if missing:
            raise ValueError("encoder checkpoint lacks: %s" % ", ".join(missing[:8]))
        assert self.layers[0].wqkv.shape == (3 * H, H)

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        self.load_state(random_bert_state(self.cfg, seed, std, self.device, self.dtype))

    def load_pretrained(self, path: str) -> None:
        from .loader import iter_safetensors_dir
        self.load_state(iter_safetensors_dir(path))

    def num_parameters(self) -> int:
        n = sum(t.numel() for t in (self.word, self.pos, self.type, self.emb_g, self.emb_b))
        for lw in self.layers:
            n += sum(getattr(lw, s).numel() for s in lw.__slots__)
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, seq_lens: Sequence[int],
                token_type_ids: Optional[torch.Tensor] = None, attn_meta=None) -> torch.Tensor:
        """Hidden states [T, H] of the packed batch."""
        cfg = self.cfg
        eps = cfg.layer_norm_eps
        Hh, D = cfg.num_attention_heads, cfg.head_dim
        H = cfg.hidden_size
        h = ops.bert_embed_ln(input_ids, positions, token_type_ids, self.word, self.pos, self.type,
                              self.emb_g, self.emb_b, eps)
        if attn_meta is None and h.is_cuda:
            attn_meta = self.attention_metadata(seq_lens)
        for lw in self.layers:
            qkv = ops.linear(h, lw.wqkv, bias=lw.bqkv)
            a = ops.attention_contiguous(qkv[:, :H], qkv[:, H:2 * H], qkv[:, 2 * H:], seq_lens, Hh, D,
                                         causal=False, meta=attn_meta)
            x = ops.linear(a, lw.wo, bias=lw.bo, residual=h)
            h = ops.layernorm(x, lw.ln1_g, lw.ln1_b, eps)
            u = ops.linear(h, lw.wi, bias=lw.bi, act="gelu")
            x = ops.linear(u, lw.wd, bias=lw.bd, residual=h)
            h = ops.layernorm(x, lw.ln2_g, lw.ln2_b, eps)
        return h

    def attention_metadata(self, seq_lens: Sequence[int]):
        cfg = self.cfg
        starts = np.concatenate([[0], np.cumsum(seq_lens)[:-1]]).astype(np.int64)
        return ops.build_attention_metadata(list(seq_lens), list(seq_lens), None, 1,
                                            cfg.num_attention_heads, cfg.head_dim, self.device,
                                            causal=False, Hkv=cfg.num_attention_heads,
                                            seq_rows=starts, allow_split=False)

    def embed(self, input_ids: torch.Tensor, positions: torch.Tensor, seq_lens: Sequence[int],
              starts: torch.Tensor, token_type_ids: Optional[torch.Tensor] = None,
              pooling: Optional[str] = None, normalize: Optional[bool] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Pooled fp32 embeddings [S, H]; ``starts`` int64 [S+1] on the model's device."""
        h = self.forward(input_ids, positions, seq_lens, token_type_ids)
        return ops.pool_normalize(h, starts, pooling or self.cfg.pooling,
                                  self.cfg.normalize if normalize is None else normalize, out=out)
