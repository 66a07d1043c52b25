"""Checkpoint formats on disk: sharded safetensors, and the three fp8 layouts found in
published checkpoints (per-channel ``weight_scale`` of compressed-tensors "FP8-dynamic"
models, per-tensor ``weight_scale`` + ``input_scale``, 128 x 128 block ``weight_scale_inv``).
Each loads to the same model as the dequantised weights given directly."""

import json
import os

import pytest
import torch

from arcticinference_b200 import LLM, SamplingParams
from arcticinference_b200.config import PRESETS
from arcticinference_b200.models.loader import random_llama_state
from arcticinference_b200.utils.safetensors_io import write_safetensors

E4M3_MAX = 448.0
LINEAR = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def _quantise(w: torch.Tensor, layout: str):
    """(codes, scale tensors by suffix, the matrix the codes stand for)."""
    wf = w.float()
    if layout == "channel":
        s = wf.abs().amax(1, keepdim=True).clamp(min=1e-12) / E4M3_MAX             # [N, 1]
        q = (wf / s).to(torch.float8_e4m3fn)
        return q, {"weight_scale": s.to(torch.bfloat16)}, q.float() * s.to(torch.bfloat16).float()
    if layout == "tensor":
        s = wf.abs().amax().clamp(min=1e-12) / E4M3_MAX
        q = (wf / s).to(torch.float8_e4m3fn)
        return q, {"weight_scale": s.reshape(()), "input_scale": torch.tensor(0.01)}, q.float() * s
    N, K = wf.shape
    blocks = wf.reshape(N // 128, 128, K // 128, 128)
    s = blocks.abs().amax((1, 3)).clamp(min=1e-12) / E4M3_MAX                       # [N/128, K/128]
    q = (blocks / s[:, None, :, None]).to(torch.float8_e4m3fn)
    deq = (q.float() * s[:, None, :, None]).reshape(N, K)
    return q.reshape(N, K), {"weight_scale_inv": s}, deq


def _write(tmp, cfg_dict, tensors: dict, shards: int = 2):
    names = list(tensors)
    per = (len(names) + shards - 1) // shards
    index = {}
    for i in range(shards):
        part = {n: tensors[n] for n in names[i * per:(i + 1) * per]}
        fname = "model-%05d-of-%05d.safetensors" % (i + 1, shards)
        write_safetensors(os.path.join(tmp, fname), part)
        index.update({n: fname for n in part})
    with open(os.path.join(tmp, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": index}, f)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg_dict, f)


def _hf_config(cfg, quant=None) -> dict:
    d = dict(architectures=[cfg.architecture], model_type=cfg.model_type, hidden_size=cfg.hidden_size,
             num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
             num_key_value_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
             intermediate_size=cfg.intermediate_size, vocab_size=cfg.vocab_size,
             rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
             max_position_embeddings=cfg.max_position_embeddings, tie_word_embeddings=False)
    if quant:
        d["quantization_config"] = quant
    return d


def _first_logits(llm):
    eng = llm.engine
    for p in ([3, 9, 27, 81, 243, 5], list(range(40, 90))):
        eng.add_request(None, p, SamplingParams(temperature=0, max_tokens=2, ignore_eos=True))
    out = eng.scheduler.schedule()
    batch, _ = eng.runner.prepare(out)
    with torch.inference_mode():
        return eng.runner.model.compute_logits(eng.runner.model.forward(batch, eng.runner.kv)).float()


QUANT_CONFIGS = {
    "channel": {"quant_method": "compressed-tensors", "format": "float-quantized",
                "ignore": ["lm_head"]},
    "tensor": {"quant_method": "fp8", "activation_scheme": "static"},
    "block": {"quant_method": "fp8", "weight_block_size": [128, 128]},
}


@pytest.mark.parametrize("layout", [None, "channel", "tensor", "block"])
def test_checkpoint_on_disk_loads_to_the_same_model(layout, tmp_path):
    cfg = PRESETS["llama-tiny"]
    state = dict(random_llama_state(cfg, seed=5, std=0.05, device="cpu", dtype=torch.bfloat16))
    on_disk, meant = {}, {}
    for name, t in state.items():
        if layout and name.endswith(".weight") and name.split(".")[-2] in LINEAR:
            q, scales, deq = _quantise(t, layout)
            on_disk[name] = q
            for sfx, s in scales.items():
                on_disk[name[:-len("weight")] + sfx] = s
            meant[name] = deq.to(torch.bfloat16)
        else:
            on_disk[name] = t
            meant[name] = t
    src, ref_dir = tmp_path / "ckpt", tmp_path / "ref"
    src.mkdir(), ref_dir.mkdir()
    _write(str(src), _hf_config(cfg, QUANT_CONFIGS.get(layout)), on_disk)
    _write(str(ref_dir), _hf_config(cfg), meant, shards=1)

    kw = dict(device="cpu", max_model_len=128, num_gpu_blocks_override=32, block_size=16)
    got = LLM(model=str(src), **kw)
    assert got.engine.config.model.quantization == ("fp8" if layout else None)
    # the oracle: the same engine over the matrices the codes stand for
    want = LLM(model=str(ref_dir), quantization="fp8" if layout else None, **kw)
    a, b = _first_logits(got), _first_logits(want)
    assert torch.equal(a, b)
    if layout == "block":
        # the default scheme re-quantises to one scale per output feature; `fp8_scheme="block"`
        # keeps the checkpoint's scheme, and re-quantising what the codes stand for on the
        # same 128 x 128 blocks gives the codes back
        kept = LLM(model=str(src), fp8_scheme="block", **kw)
        same = LLM(model=str(ref_dir), quantization="fp8", fp8_scheme="block", **kw)
        c, d = _first_logits(kept), _first_logits(same)
        assert (c - d).abs().max().item() <= 0.02 * max(1.0, d.abs().max().item())
        w = kept.engine.runner.model.layers[0].wdown
        deq = meant["model.layers.0.mlp.down_proj.weight"].float()
        assert (w.dequantize().float() - deq).abs().max().item() <= 0.01 * deq.abs().max().item()
