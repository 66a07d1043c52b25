"""Helpers shared by the sending and receiving side: the HF-named view of an engine's weights
(what a trainer must send, and what the engine can send back), in-place re-quantisation of
fp8 weights, and a checksum.
(reference: arctic_inference/server/weight_sync/utils.py:166-294 fp8 in-place requant,
:32-79 rendezvous; receiver.py:130-190 weights info.)
"""

from __future__ import annotations

from typing import Iterator

import torch

from .schedule import TensorMeta, dtype_name

DIRECT_NAMES = ("model.embed_tokens.weight", "lm_head.weight", "model.norm.weight",
                "model.norm_swiftkv.weight")


def expected_llama_tensors(cfg, dtype: torch.dtype = torch.bfloat16) -> list[TensorMeta]:
    """Names, full (unsharded) shapes and dtype of the checkpoint tensors a Llama / SwiftKV
    engine consumes."""
    H, D = cfg.hidden_size, cfg.head_dim
    Hq, I = cfg.num_attention_heads, cfg.intermediate_size
    Hkv = cfg.checkpoint_kv_heads or cfg.num_key_value_heads     # the trainer's shapes
    dn = dtype_name(dtype)
    out = [TensorMeta("model.embed_tokens.weight", (cfg.vocab_size, H), dn, True),
           TensorMeta("model.norm.weight", (H,), dn, True)]
    if cfg.tie_word_embeddings:
        out.append(TensorMeta("lm_head.weight", (cfg.vocab_size, H), dn, False,
                              alias_of="model.embed_tokens.weight"))
    else:
        out.append(TensorMeta("lm_head.weight", (cfg.vocab_size, H), dn, True))
    if cfg.is_swiftkv:
        out.append(TensorMeta("model.norm_swiftkv.weight", (H,), dn, True))
    for l in range(cfg.num_hidden_layers):
        p = "model.layers.%d." % l
        sfx = "_swiftkv" if cfg.is_swiftkv and l >= cfg.num_key_value_layers else ""
        out += [TensorMeta(p + "input_layernorm.weight", (H,), dn),
                TensorMeta(p + "post_attention_layernorm.weight", (H,), dn),
                TensorMeta(p + "self_attn.q_proj%s.weight" % sfx, (Hq * D, H), dn),
                TensorMeta(p + "self_attn.k_proj%s.weight" % sfx, (Hkv * D, H), dn),
                TensorMeta(p + "self_attn.v_proj%s.weight" % sfx, (Hkv * D, H), dn),
                TensorMeta(p + "self_attn.o_proj.weight", (H, Hq * D), dn),
                TensorMeta(p + "mlp.gate_proj.weight", (I, H), dn),
                TensorMeta(p + "mlp.up_proj.weight", (I, H), dn),
                TensorMeta(p + "mlp.down_proj.weight", (H, I), dn)]
        if cfg.qk_norm:
            out += [TensorMeta(p + "self_attn.q_norm.weight", (D,), dn),
                    TensorMeta(p + "self_attn.k_norm.weight", (D,), dn)]
        if cfg.qkv_bias:
            out += [TensorMeta(p + "self_attn.q_proj.bias", (Hq * D,), dn),
                    TensorMeta(p + "self_attn.k_proj.bias", (Hkv * D,), dn),
                    TensorMeta(p + "self_attn.v_proj.bias", (Hkv * D,), dn)]
    return out


def _dense(w) -> torch.Tensor:
    return w if isinstance(w, torch.Tensor) else w.dequantize()


def export_llama_state(model) -> Iterator:
    """(name, tensor) pairs in checkpoint naming rebuilt from the fused engine weights. Needs
    a rank that stores every head block (a single-GPU replica)."""
    cfg = model.cfg
    blocks = list(model.shard.stored_blocks)
    if len(blocks) != model.shard.ways:
        raise NotImplementedError("exporting checkpoint-named weights needs a single-GPU replica; "
                                  "this rank stores %d of %d head blocks" % (len(blocks), model.shard.ways))
    D, h, hkv, Ib = model.D, model.h, model.hkv, model.inter_blk
    yield "model.embed_tokens.weight", model.embed
    yield "model.norm.weight", model.norm
    if not cfg.tie_word_embeddings:
        yield "lm_head.weight", model.lm_head
    if cfg.is_swiftkv:
        yield "model.norm_swiftkv.weight", model.norm_swiftkv
    n_later = cfg.num_hidden_layers - model.n_kv_layers
    wkv = _dense(model.wkv_swiftkv) if model.wkv_swiftkv is not None else None
    for l, lw in enumerate(model.layers):
        p = "model.layers.%d." % l
        later = cfg.is_swiftkv and l >= model.n_kv_layers
        sfx = "_swiftkv" if later else ""
        qkv, gu = _dense(lw.wqkv), _dense(lw.wgu)
        rows = (h + 2 * hkv) * D
        qs, ks, vs, gs, us = [], {}, {}, [], []
        for i, b in enumerate(blocks):
            blk = qkv[i * rows:(i + 1) * rows]
            qs.append(blk[:h * D])
            kvh = model.kv_head_of_block(b)
            ks[kvh.start] = blk[h * D:(h + hkv) * D]
            vs[kvh.start] = blk[(h + hkv) * D:]
            g = gu[i * 2 * Ib:(i + 1) * 2 * Ib]
            gs.append(g[:Ib])
            us.append(g[Ib:])
        if later:
            # the later layers' K/V projections live in the fused SwiftKV matrix
            width = 2 * hkv * D
            j = l - model.n_kv_layers
            for i, b in enumerate(blocks):
                kvh = model.kv_head_of_block(b)
                r0 = i * n_later * width + j * width
                ks[kvh.start] = wkv[r0:r0 + hkv * D]
                vs[kvh.start] = wkv[r0 + hkv * D:r0 + width]
        yield p + "input_layernorm.weight", lw.input_norm
        yield p + "post_attention_layernorm.weight", lw.post_norm
        if lw.q_norm is not None:
            yield p + "self_attn.q_norm.weight", lw.q_norm
            yield p + "self_attn.k_norm.weight", lw.k_norm
        if lw.bqkv is not None:
            bq, bk, bv = [], {}, {}
            for i, b in enumerate(blocks):
                blk = lw.bqkv[i * rows:(i + 1) * rows]
                kvh = model.kv_head_of_block(b)
                bq.append(blk[:h * D])
                bk[kvh.start] = blk[h * D:(h + hkv) * D]
                bv[kvh.start] = blk[(h + hkv) * D:]
            yield p + "self_attn.q_proj.bias", torch.cat(bq, 0)
            yield p + "self_attn.k_proj.bias", _checkpoint_heads(cfg, [bk[k] for k in sorted(bk)])
            yield p + "self_attn.v_proj.bias", _checkpoint_heads(cfg, [bv[k] for k in sorted(bv)])
        yield p + "self_attn.q_proj%s.weight" % sfx, torch.cat(qs, 0)
        yield p + "self_attn.k_proj%s.weight" % sfx, _checkpoint_heads(cfg, [ks[k] for k in sorted(ks)])
        yield p + "self_attn.v_proj%s.weight" % sfx, _checkpoint_heads(cfg, [vs[k] for k in sorted(vs)])
        yield p + "self_attn.o_proj.weight", _dense(lw.wo)
        yield p + "mlp.gate_proj.weight", torch.cat(gs, 0)
        yield p + "mlp.up_proj.weight", torch.cat(us, 0)
        yield p + "mlp.down_proj.weight", _dense(lw.wdown)


def _checkpoint_heads(cfg, parts: list) -> torch.Tensor:
    """Stored K/V heads back to the checkpoint's: one of every ``kv_head_replication``."""
    w = torch.cat(parts, 0)
    r, D = cfg.kv_head_replication, cfg.head_dim
    if r == 1:
        return w
    return w.reshape(-1, r, D, *w.shape[1:])[:, 0].reshape(-1, *w.shape[1:])


def requantize_into(dst, dense: torch.Tensor) -> None:
    """Overwrite an fp8 weight in place with the re-quantised ``dense`` matrix (codes, scales
    and a bf16 prefill shadow keep their addresses, so captured graphs stay valid)."""
    dst.requantize_from(dense)


def assign_in_place(dst, src: torch.Tensor):
    """Copy ``src`` into the engine weight ``dst`` (tensor or fp8 weight)."""
    if isinstance(dst, torch.Tensor):
        dst.copy_(src.to(dst.dtype))
    else:
        requantize_into(dst, src)
    return dst


def engine_weight_norm(engine) -> float:
    """L2 norm over every weight this rank stores (fp8 weights are expanded): a cheap check
    that two replicas, or a replica and the trainer, hold the same parameters."""
    m = engine.runner.model
    acc = torch.zeros((), dtype=torch.float64, device=m.device)
    ts = [m.embed, m.norm, m.norm_swiftkv, m.wkv_swiftkv]
    if m.lm_head is not m.embed:
        ts.append(m.lm_head)
    for lw in m.layers:
        ts += [t for _, t in lw.tensors()]
    for t in ts:
        if t is None:
            continue
        acc += _dense(t).double().pow(2).sum()
    return float(acc.sqrt())
