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
                 "kv_bulk_write", "kv_write_fp4"):
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
