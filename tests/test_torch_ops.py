"""``torch.ops.arcticinference_b200``: the library builds and registers its schemas (CPU);
on a GPU every op returns what the engine's own entry points return."""

import pytest
import torch

from arcticinference_b200 import build


@pytest.fixture(scope="module")
def tops():
    return build.load_torch_ops()


def test_schemas_registered(tops):
    for name in ("linear", "rmsnorm", "silu_mul", "spec_ln", "mlp_spec_step", "sum_lstm",
                 "kv_bulk_write", "kv_write_fp4", "quant_fp8_row", "rmsnorm_quant",
                 "silu_mul_quant", "linear_fp8_row", "rope_cache", "attention"):
        assert hasattr(tops, name)
    s = str(tops.sum_lstm.default._schema)
    assert "Tensor gates" in s and "-> (Tensor, Tensor)" in s
    with pytest.raises((NotImplementedError, RuntimeError)):
        tops.silu_mul(torch.zeros(2, 8, dtype=torch.bfloat16), 1)        # no CPU kernel


@pytest.mark.gpu
def test_ops_match_engine_entry_points(tops):
    from arcticinference_b200 import ops
    from arcticinference_b200.ops import spec_ops
    dev = "cuda:0"
    R = lambda *s, sc=1.0: (torch.randn(*s, device=dev) * sc).to(torch.bfloat16)
    x, w, b, res = R(70, 512), R(384, 512, sc=0.05), R(384), R(70, 384)
    assert torch.equal(tops.linear(x, w, b, res, 1), ops.linear(x, w, bias=b, residual=res, act="gelu"))
    g = R(512)
    r1, r2 = R(70, 512), None
    r2 = r1.clone()
    assert torch.equal(tops.rmsnorm(x, g, 1e-5, r1), ops.rmsnorm(x, g, 1e-5, residual=r2)) and torch.equal(r1, r2)
    gu = R(33, 2 * 256)
    assert torch.equal(tops.silu_mul(gu, 1), ops.silu_mul(gu))
    assert torch.equal(tops.spec_ln(x, g, None, 1e-6, 0.5), spec_ops.spec_ln(x, g, None, 1e-6, 0.5))
    D, V, B = 256, 100, 9
    gates, emb, tok = R(B, 4 * D), R(V, D), torch.randint(0, V, (B,), device=dev)
    wc, ws = 1 + R(D, sc=0.1), 1 + R(D, sc=0.1)
    c1, h1 = tops.sum_lstm(gates, emb, tok, 0.7, None, wc, None, ws, None, 1e-6, False)
    c2, h2 = spec_ops.sum_lstm(gates, emb, tok, 0.7, None, wc, None, ws, None, 1e-6)
    assert torch.equal(c1, c2) and torch.equal(h1, h2)
    c3, h3 = tops.sum_lstm(gates, emb, tok, 0.7, c1, wc, None, ws, None, 1e-6, False)
    c4, h4 = spec_ops.sum_lstm(gates, emb, tok, 0.7, c2, wc, None, ws, None, 1e-6)
    assert torch.equal(c3, c4) and torch.equal(h3, h4)
    proj = R(B, D)
    assert torch.equal(tops.mlp_spec_step(proj, emb, tok, 0.3, wc, None, 1e-6, False),
                       spec_ops.mlp_spec_step(proj, emb, tok, 0.3, wc, None, 1e-6))
    # cache writers
    T, L, Hkv, Dh, bs, nb = 11, 3, 2, 128, 16, 4
    kv = R(T, L * 2 * Hkv * Dh)
    pos = torch.arange(T, device=dev)
    slots = torch.randperm(nb * bs, device=dev)[:T]
    inv = 1.0 / (10000.0 ** (torch.arange(0, Dh, 2, device=dev).float() / Dh))
    mk = lambda: [torch.zeros(nb, Hkv, bs, Dh, device=dev, dtype=torch.bfloat16) for _ in range(L)]
    k1, v1, k2, v2 = mk(), mk(), mk(), mk()
    ptr = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    tops.kv_bulk_write(kv, pos, slots, inv, ptr(k1), ptr(v1), None, None, Hkv, Dh, bs, nb * bs, False)
    ops.kv_bulk_write(kv, pos, slots, inv, k2, v2, Hkv, Dh)
    assert all(torch.equal(a, b) for a, b in zip(k1 + v1, k2 + v2))
    k, v = R(T, Hkv * Dh), R(T, Hkv * Dh)
    mk4 = lambda last: torch.zeros(nb, Hkv, bs, last, device=dev, dtype=torch.uint8)
    a = [mk4(Dh // 2), mk4(Dh // 2), mk4(Dh // 16), mk4(Dh // 16)]
    b4 = [t.clone() for t in a]
    tops.kv_write_fp4(k, v, slots, *a)
    ops.kv_write_fp4(k, v, slots, *b4, Hkv, Dh)
    assert all(torch.equal(p, q) for p, q in zip(a, b4))
    ops.check_status()


@pytest.mark.gpu
def test_fp8_and_attention_ops_match_engine_entry_points(tops):
    import math
    from arcticinference_b200 import ops
    from arcticinference_b200.models import quant
    dev = "cuda:0"
    R = lambda *s, sc=1.0: (torch.randn(*s, device=dev) * sc).to(torch.bfloat16)
    same = lambda a, b: torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    x, g = R(70, 512), 1 + R(512, sc=0.1)
    q, sx = tops.quant_fp8_row(x)
    want = ops.quant_fp8_row(x)
    assert same(q, want.q) and torch.equal(sx, want.scale)
    r1, r2 = R(70, 512), None
    r2 = r1.clone()
    q1, s1 = tops.rmsnorm_quant(x, g, 1e-5, r1)
    want = ops.rmsnorm(x, g, 1e-5, residual=r2, quant=True)
    assert same(q1, want.q) and torch.equal(s1, want.scale) and torch.equal(r1, r2)
    gu = R(33, 2 * 256)
    q2, s2 = tops.silu_mul_quant(gu, 1)
    want = ops.silu_mul_blocked(gu, 1, quant=True)
    assert same(q2, want.q) and torch.equal(s2, want.scale)
    w = quant.quantize_weight_fp8_row(R(384, 512, sc=0.05), tiled=False)
    b, res = R(384), R(70, 384)
    got = tops.linear_fp8_row(q, sx, w.q, w.scale, b, res, 0)
    assert torch.equal(got, ops.linear(quant.QuantAct(q, sx), w, bias=b, residual=res))
    # RoPE + cache write, then paged attention over the written cache
    Hq, Hkv, D, bs, nb = 8, 2, 128, 16, 12
    q_lens, kv_lens = [5, 1, 40], [5, 9, 40]
    T = sum(q_lens)
    qkv = R(T, (Hq + 2 * Hkv) * D)
    qkv2 = qkv.clone()
    pos = torch.cat([torch.arange(k - n, k) for n, k in zip(q_lens, kv_lens)]).to(dev)
    bt = torch.zeros(3, 4, dtype=torch.int32)
    bt[0, :1], bt[1, :1], bt[2, :3] = torch.tensor([1]), torch.tensor([2]), torch.tensor([3, 4, 5])
    slots = torch.cat([bt[i, p // bs].long() * bs + p % bs
                       for i, (n, k) in enumerate(zip(q_lens, kv_lens))
                       for p in [torch.arange(k - n, k)]]).to(dev)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
    mk = lambda: torch.zeros(nb, Hkv, bs, D, device=dev, dtype=torch.bfloat16)
    k1, v1, k2, v2 = mk(), mk(), mk(), mk()
    tops.rope_cache(qkv, pos, slots, inv, k1, v1, Hq, Hkv, D)
    ops.rope_cache(qkv2, pos, slots, inv, k2, v2, Hq, Hkv, D)
    assert torch.equal(qkv, qkv2) and torch.equal(k1, k2) and torch.equal(v1, v2)
    meta = ops.build_attention_metadata(q_lens, kv_lens, bt.to(dev), Hq // Hkv, Hq, D, dev, Hkv=Hkv)
    qq = qkv[:, :Hq * D]
    want = ops.attention(qq, k1, v1, meta, Hq, Hkv, D, 1 / math.sqrt(D))
    got = tops.attention(qq, k1, v1, meta.block_tables, meta.work, meta.tok_splits,
                         meta.max_splits, Hq, Hkv, D, True, 1 / math.sqrt(D), meta.tile_keys)
    assert torch.equal(got, want)
    ops.check_status()
