"""Encoder kernels and the embedding engine on the GPU, against fp32 PyTorch restatements."""

import numpy as np
import pytest
import torch

from arcticinference_b200 import ops
from arcticinference_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("H", [128, 768, 1024])
def test_bert_embed_ln(H):
    T, V, P = 45, 500, 64
    word, pos, typ = _rand(V, H, scale=0.05), _rand(P, H, scale=0.05), _rand(2, H, scale=0.05)
    g, b = 1 + _rand(H, scale=0.1), _rand(H, scale=0.1)
    ids = torch.randint(0, V, (T,), device=DEV)
    p = torch.randint(0, P, (T,), device=DEV)
    ty = torch.randint(0, 2, (T,), device=DEV)
    for t in (ty, None):
        y = ops.bert_embed_ln(ids, p, t, word, pos, typ, g, b, 1e-12)
        want = ref.bert_embed_ln(ids, p, t, word.float(), pos.float(), typ.float(), g, b, 1e-12)
        ops.check_status()
        assert float((y.float() - want.float()).abs().max()) < 4e-2


@pytest.mark.parametrize("mode", ["cls", "mean", "last"])
@pytest.mark.parametrize("normalize", [True, False])
def test_pool_normalize(mode, normalize):
    H = 768
    lens = [1, 50, 512, 7]
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int64, device=DEV)
    h = _rand(sum(lens), H)
    y = ops.pool_normalize(h, starts, mode, normalize)
    want = ref.pool_normalize(h, starts.cpu(), mode, normalize)
    assert y.dtype == torch.float32
    assert float((y - want).abs().max()) < 2e-3


def test_embedding_engine_matches_cpu_oracle():
    from arcticinference_b200.embedding.engine import EmbeddingEngine
    gpu = EmbeddingEngine("bert-tiny", device=DEV, max_num_batched_tokens=1024, max_num_seqs=16)
    cpu = EmbeddingEngine("bert-tiny", device="cpu", dtype=torch.float32,
                          max_num_batched_tokens=1024, max_num_seqs=16)
    # same weights on both sides (the two devices' random generators differ)
    from arcticinference_b200.models.bert import random_bert_state
    gpu.encoder.load_state(random_bert_state(gpu.cfg, 0, 0.05, "cpu", torch.float32))
    cpu.encoder.load_state(random_bert_state(cpu.cfg, 0, 0.05, "cpu", torch.float32))
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 1000, size=n).tolist() for n in
            [50, 512, 1, 129, 128, 300, 64, 3, 200, 77, 50, 50, 50, 400, 31, 2, 90, 250]]
    before = ops.launch_counter.n
    a = gpu.encode(seqs)
    assert ops.launch_counter.n > before                  # the CUDA kernels ran
    b = cpu.encode(seqs)
    cos = (a * b).sum(1)
    assert float(cos.min()) > 0.995, float(cos.min())
    assert np.allclose(np.linalg.norm(a, axis=1), 1.0, atol=1e-3)
    m = gpu.encode(seqs[:4], pooling="mean")
    mc = cpu.encode(seqs[:4], pooling="mean")
    assert float((m * mc).sum(1).min()) > 0.995


def test_bert_base_shapes_run():
    from arcticinference_b200.embedding.engine import EmbeddingEngine
    e = EmbeddingEngine("bert-base", device=DEV)
    rng = np.random.default_rng(1)
    seqs = [rng.integers(0, 30522, size=n).tolist() for n in [50] * 40 + [512] * 6]
    v = e.encode(seqs)
    assert v.shape == (46, 768) and np.isfinite(v).all()
    again = e.encode(seqs[::-1])[::-1]
    assert np.allclose(v, again, atol=2e-2)
