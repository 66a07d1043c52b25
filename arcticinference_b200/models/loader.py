"""Checkpoint names -> packed, sharded engine weights.

Accepted formats (reference: arctic_inference/vllm/swiftkv/llama_swiftkv.py:748-820,
arctic_inference/vllm/spec_dec/fp8.py:140-180):

* Hugging Face Llama / Mistral / Qwen2 / Qwen3 safetensors (``q_proj/k_proj/v_proj/o_proj``,
  ``gate_proj/up_proj/down_proj``, norms, ``embed_tokens``, ``lm_head``; for Qwen2 also the
  ``q_proj/k_proj/v_proj`` biases, for Qwen3 ``self_attn.q_norm`` and ``self_attn.k_norm``);
* SwiftKV: ``model_type = llama_swiftkv``, ``num_key_value_layers`` and, for each layer
  >= num_key_value_layers, ``self_attn.{q,k,v}_proj_swiftkv`` plus ``model.norm_swiftkv``;
* fp8 checkpoints: fp8 ``weight`` with a per-tensor / per-channel ``weight_scale`` or a
  128x128-block ``weight_scale_inv``. They are expanded to bf16 while packing; because
  every packed block boundary is a multiple of 128 rows, re-quantising the packed matrix
  on 128x128 blocks reproduces the checkpoint's codes.

Packing turns the per-projection matrices into the rank-major fused layout of
:mod:`.llama` and keeps only the head blocks this rank stores.
"""

from __future__ import annotations

import glob
import os
import re
from typing import Iterable, Iterator

import torch

_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")


def random_llama_state(cfg, seed: int, std: float, device, dtype) -> Iterator:
    """Yield (name, tensor) pairs of a random checkpoint in Hugging Face naming."""
    gen = torch.Generator(device=device)
    H, D = cfg.hidden_size, cfg.head_dim
    Hq, Hkv, I = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size

    def rnd(tag, *shape):
        gen.manual_seed(seed * 1000003 + tag)
        return (torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)

    ones = lambda: torch.ones(H, device=device, dtype=dtype)
    yield "model.embed_tokens.weight", rnd(1, cfg.vocab_size, H)
    if not cfg.tie_word_embeddings:
        yield "lm_head.weight", rnd(2, cfg.vocab_size, H)
    yield "model.norm.weight", ones()
    if cfg.is_swiftkv:
        yield "model.norm_swiftkv.weight", ones()
    for l in range(cfg.num_hidden_layers):
        p = "model.layers.%d." % l
        b = 100 + 20 * l
        yield p + "input_layernorm.weight", ones()
        yield p + "post_attention_layernorm.weight", ones()
        if cfg.qkv_bias:
            yield p + "self_attn.q_proj.bias", 5 * rnd(b + 10, Hq * D)
            yield p + "self_attn.k_proj.bias", 5 * rnd(b + 11, Hkv * D)
            yield p + "self_attn.v_proj.bias", 5 * rnd(b + 12, Hkv * D)
        if cfg.qk_norm:
            yield p + "self_attn.q_norm.weight", (1.0 + 10 * rnd(b + 8, D).float()).to(dtype)
            yield p + "self_attn.k_norm.weight", (1.0 + 10 * rnd(b + 9, D).float()).to(dtype)
        later = cfg.is_swiftkv and l >= cfg.num_key_value_layers
        sfx = "_swiftkv" if later else ""
        yield p + "self_attn.q_proj%s.weight" % sfx, rnd(b + 1, Hq * D, H)
        yield p + "self_attn.k_proj%s.weight" % sfx, rnd(b + 2, Hkv * D, H)
        yield p + "self_attn.v_proj%s.weight" % sfx, rnd(b + 3, Hkv * D, H)
        yield p + "self_attn.o_proj.weight", rnd(b + 4, H, Hq * D)
        yield p + "mlp.gate_proj.weight", rnd(b + 5, I, H)
        yield p + "mlp.up_proj.weight", rnd(b + 6, I, H)
        yield p + "mlp.down_proj.weight", rnd(b + 7, H, I)


def _expand_fp8(weight: torch.Tensor, scale: torch.Tensor, inverse_block: bool) -> torch.Tensor:
    w = weight.float()
    s = scale.float()
    if inverse_block and s.dim() == 2 and s.shape != w.shape:
        bn = (w.shape[0] + s.shape[0] - 1) // s.shape[0]
        bk = (w.shape[1] + s.shape[1] - 1) // s.shape[1]
        s = s.repeat_interleave(bn, 0)[: w.shape[0]].repeat_interleave(bk, 1)[:, : w.shape[1]]
    elif s.dim() == 1 and s.numel() == w.shape[0]:
        s = s.unsqueeze(1)
    return (w * s).to(torch.bfloat16)


def expand_kv_heads(cfg, w: torch.Tensor) -> torch.Tensor:
    """K or V projection rows (or bias) of the checkpoint's heads -> of the heads the engine
    stores: each head ``cfg.kv_head_replication`` times in a row (a tensor that already has
    the stored number of heads passes through)."""
    r, D = cfg.kv_head_replication, cfg.head_dim
    if r == 1 or w.shape[0] == cfg.num_key_value_heads * D:
        return w
    if w.shape[0] != cfg.checkpoint_kv_heads * D:
        raise ValueError("K/V projection with %d rows; expected %d heads of %d" %
                         (w.shape[0], cfg.checkpoint_kv_heads, D))
    heads = w.reshape(cfg.checkpoint_kv_heads, D, *w.shape[1:])
    return heads.repeat_interleave(r, dim=0).reshape(-1, *w.shape[1:])


def _required(model, l: int) -> list[str]:
    later = model.cfg.is_swiftkv and l >= model.n_kv_layers
    sfx = "_swiftkv" if later else ""
    norms = ["self_attn.q_norm.weight", "self_attn.k_norm.weight"] if model.cfg.qk_norm else []
    if model.cfg.qkv_bias:
        norms += ["self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias"]
    return ["input_layernorm.weight", "post_attention_layernorm.weight",
            "self_attn.q_proj%s.weight" % sfx, "self_attn.k_proj%s.weight" % sfx,
            "self_attn.v_proj%s.weight" % sfx, "self_attn.o_proj.weight",
            "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"] + norms


def pack_llama_layer(model, l: int, t: dict) -> None:
    """Build layer ``l``'s fused tensors from per-projection matrices (all on any device)."""
    from .llama import LlamaLayerWeights
    dev, dt = model.device, model.dtype
    D, h, hkv, Ib = model.D, model.h, model.hkv, model.inter_blk
    later = model.cfg.is_swiftkv and l >= model.n_kv_layers
    sfx = "_swiftkv" if later else ""
    q = t["self_attn.q_proj%s.weight" % sfx]
    k = expand_kv_heads(model.cfg, t["self_attn.k_proj%s.weight" % sfx])
    v = expand_kv_heads(model.cfg, t["self_attn.v_proj%s.weight" % sfx])
    if model.cfg.qkv_bias:
        t = dict(t)
        for name in ("self_attn.k_proj.bias", "self_attn.v_proj.bias"):
            t[name] = expand_kv_heads(model.cfg, t[name])
    gate, up = t["mlp.gate_proj.weight"], t["mlp.up_proj.weight"]
    blocks = list(model.shard.stored_blocks)
    lw = LlamaLayerWeights()
    qkv_rows, gu_rows, kv_rows, bias_rows = [], [], [], []
    for p in blocks:
        kvh = model.kv_head_of_block(p)
        ks = k[kvh.start * D: kvh.stop * D]
        vs = v[kvh.start * D: kvh.stop * D]
        qkv_rows += [q[p * h * D:(p + 1) * h * D], ks, vs]
        if model.cfg.qkv_bias:
            bias_rows += [t["self_attn.q_proj.bias"][p * h * D:(p + 1) * h * D],
                          t["self_attn.k_proj.bias"][kvh.start * D: kvh.stop * D],
                          t["self_attn.v_proj.bias"][kvh.start * D: kvh.stop * D]]
        gu_rows += [gate[p * Ib:(p + 1) * Ib], up[p * Ib:(p + 1) * Ib]]
        kv_rows.append((ks, vs))
    to = lambda x: x.to(device=dev, dtype=dt)
    lw.wqkv = to(torch.cat(qkv_rows, 0)).contiguous()
    lw.wgu = to(torch.cat(gu_rows, 0)).contiguous()
    p0, n = blocks[0], len(blocks)
    lw.wo = to(t["self_attn.o_proj.weight"][:, p0 * h * D:(p0 + n) * h * D]).contiguous()
    lw.wdown = to(t["mlp.down_proj.weight"][:, p0 * Ib:(p0 + n) * Ib]).contiguous()
    lw.input_norm = to(t["input_layernorm.weight"]).contiguous()
    lw.post_norm = to(t["post_attention_layernorm.weight"]).contiguous()
    if bias_rows:
        lw.bqkv = to(torch.cat(bias_rows, 0)).contiguous()
    if model.cfg.qk_norm:
        lw.q_norm = to(t["self_attn.q_norm.weight"]).contiguous()
        lw.k_norm = to(t["self_attn.k_norm.weight"]).contiguous()
    model.layers[l] = lw
    if later:
        n_later = model.cfg.num_hidden_layers - model.n_kv_layers
        width = 2 * hkv * D
        rows_blk = n_later * width
        if model.wkv_swiftkv is None:
            model.wkv_swiftkv = torch.zeros(len(blocks) * rows_blk, model.cfg.hidden_size,
                                            device=dev, dtype=dt)
        j = l - model.n_kv_layers
        for i, (ks, vs) in enumerate(kv_rows):
            r0 = i * rows_blk + j * width
            model.wkv_swiftkv[r0:r0 + hkv * D] = to(ks)
            model.wkv_swiftkv[r0 + hkv * D:r0 + width] = to(vs)


def load_llama_state(model, state: Iterable) -> None:
    """Consume (name, tensor) pairs in checkpoint naming; tensors may arrive in any order."""
    cfg = model.cfg
    dev, dt = model.device, model.dtype
    model.layers = [None] * cfg.num_hidden_layers
    model.wkv_swiftkv = None
    pending: dict[int, dict] = {}
    scales: dict[str, tuple] = {}
    raw_fp8: dict[str, torch.Tensor] = {}

    def deliver(name: str, tensor: torch.Tensor) -> None:
        if name.startswith("speculator."):
            return
        if name == "model.embed_tokens.weight":
            model.embed = tensor.to(device=dev, dtype=dt).contiguous()
            if cfg.tie_word_embeddings:
                model.lm_head = model.embed
        elif name == "lm_head.weight":
            if not cfg.tie_word_embeddings:
                model.lm_head = tensor.to(device=dev, dtype=dt).contiguous()
        elif name == "model.norm.weight":
            model.norm = tensor.to(device=dev, dtype=dt).contiguous()
        elif name == "model.norm_swiftkv.weight":
            model.norm_swiftkv = tensor.to(device=dev, dtype=dt).contiguous()
        else:
            m = _LAYER_RE.match(name)
            if not m:
                return
            l, key = int(m.group(1)), m.group(2)
            if l >= cfg.num_hidden_layers:
                return
            if not (getattr(model, "layer_lo", 0) <= l < getattr(model, "layer_hi", l + 1)):
                return      # another pipeline stage's layer
            d = pending.setdefault(l, {})
            d[key] = tensor
            if all(r in d for r in _required(model, l)):
                pack_llama_layer(model, l, d)
                del pending[l]

    for name, tensor in state:
        if name.endswith(".weight_scale_inv") or name.endswith(".weight_scale"):
            base = name.rsplit(".", 1)[0] + ".weight"
            inv = name.endswith("_inv")
            if base in raw_fp8:
                deliver(base, _expand_fp8(raw_fp8.pop(base), tensor, inv))
            else:
                scales[base] = (tensor, inv)
            continue
        if name.endswith(("input_scale", "k_scale", "v_scale", "kv_scale")):
            continue
        if tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            if name in scales:
                s, inv = scales.pop(name)
                deliver(name, _expand_fp8(tensor, s, inv))
            else:
                raw_fp8[name] = tensor
            continue
        deliver(name, tensor)

    lo, hi = getattr(model, "layer_lo", 0), getattr(model, "layer_hi", cfg.num_hidden_layers)
    missing = [l for l, lw in enumerate(model.layers) if lw is None and lo <= l < hi]
    if missing or model.embed is None or model.norm is None:
        raise ValueError("checkpoint is incomplete: layers %s, embed=%s, norm=%s" %
                         (missing[:8], model.embed is not None, model.norm is not None))
    if model.lm_head is None:
        model.lm_head = model.embed
    if cfg.is_swiftkv and (model.norm_swiftkv is None or model.wkv_swiftkv is None):
        raise ValueError("SwiftKV checkpoint lacks norm_swiftkv / *_proj_swiftkv tensors")


def iter_safetensors_dir(path: str) -> Iterator:
    """(name, tensor) pairs of every ``*.safetensors`` file under ``path`` (or
    ``pytorch_model*.bin`` when there are none)."""
    from ..utils.safetensors_io import read_safetensors
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        for f in files:
            yield from read_safetensors(f)
        return
    for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
        sd = torch.load(f, map_location="cpu", weights_only=True)
        yield from sd.items()


def load_llama_weights(model, path: str) -> None:
    load_llama_state(model, iter_safetensors_dir(path))


class LlamaWeightUpdater:
    """In-place update of a loaded model from a stream of checkpoint-named tensors.

    ``deliver`` may be called in any order; as soon as every projection of a decoder layer
    has arrived the layer's fused, sharded tensors are rebuilt and copied *into the existing
    storage* (fp8 weights are re-quantised in place), so addresses captured in CUDA graphs or
    registered with peers stay valid. The streamed tensors may be views of a transfer buffer
    that is about to be reused: whatever has to outlive the call is copied first.
    (reference: arctic_inference/server/weight_sync/receiver.py:280-331,
    utils.py:166-294.)
    """

    def __init__(self, model):
        self.model = model
        self.pending: dict[int, dict] = {}
        self.applied = 0
        self.layers_done: set = set()
        self._wkv_stage = None

    def direct_target(self, name: str):
        """Destination tensor when ``name`` can be received straight into engine storage."""
        m = self.model
        t = {"model.embed_tokens.weight": m.embed, "model.norm.weight": m.norm,
             "model.norm_swiftkv.weight": m.norm_swiftkv,
             "lm_head.weight": None if m.lm_head is m.embed else m.lm_head}.get(name)
        return t if isinstance(t, torch.Tensor) else None

    def deliver(self, name: str, tensor) -> None:
        from ..server.weight_sync.utils import assign_in_place
        m = self.model
        if tensor is None or isinstance(tensor, str):
            self.applied += 1            # tied tensor: shares storage with its target already
            return
        direct = self.direct_target(name)
        if direct is not None:
            if tensor.data_ptr() != direct.data_ptr():
                direct.copy_(tensor.to(direct.dtype))
            self.applied += 1
            return
        if name == "lm_head.weight":     # tied in the engine, sent separately: ignore
            self.applied += 1
            return
        mt = _LAYER_RE.match(name)
        if not mt:
            return
        l, key = int(mt.group(1)), mt.group(2)
        if l >= m.cfg.num_hidden_layers:
            return
        d = self.pending.setdefault(l, {})
        d[key] = tensor.clone()          # the transfer buffer is recycled before the layer is complete
        self.applied += 1
        if all(r in d for r in _required(m, l)):
            self._apply_layer(l, d)
            del self.pending[l]

    def _apply_layer(self, l: int, d: dict) -> None:
        from ..server.weight_sync.utils import assign_in_place
        from .quant import Fp8Weight
        m = self.model
        old = m.layers[l]
        later = m.cfg.is_swiftkv and l >= m.n_kv_layers
        real_wkv = m.wkv_swiftkv
        if later and isinstance(real_wkv, Fp8Weight):
            # pack into a dense staging copy; re-quantised once at the end
            if self._wkv_stage is None:
                self._wkv_stage = real_wkv.dequantize()
            m.wkv_swiftkv = self._wkv_stage
        try:
            pack_llama_layer(m, l, d)    # builds fresh fused tensors (and writes wkv rows in place)
        finally:
            m.wkv_swiftkv = real_wkv
        new = m.layers[l]
        for slot, tensor in new.tensors():
            assign_in_place(getattr(old, slot), tensor)
        m.layers[l] = old
        self.layers_done.add(l)

    def finish(self) -> dict:
        from ..server.weight_sync.utils import requantize_into
        if self._wkv_stage is not None:
            requantize_into(self.model.wkv_swiftkv, self._wkv_stage)
            self._wkv_stage = None
        incomplete = sorted(self.pending)
        self.pending = {}
        return {"tensors": self.applied, "layers": len(self.layers_done),
                "incomplete_layers": incomplete}
