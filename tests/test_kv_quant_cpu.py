"""CPU checks of the NVFP4 quantiser oracle and of the CPU paths of the KV-cache writers."""

import torch

from arcticinference_b200 import ops
from arcticinference_b200.ops import reference as ref


def test_nvfp4_oracle_values():
    x = torch.tensor([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -6.0, -0.5, 0.25, 0.75, 1.25, 2.5,
                       3.5, 5.0]])
    codes, scales, deq = ref.quantize_nvfp4(x)
    assert float(scales.view(torch.float8_e4m3fn).float()) == 1.0       # amax 6 -> scale 1
    # exact grid points survive; ties go to the even code: .25->0, .75->1, 1.25->1, 2.5->2,
    # 3.5->4, 5->4
    want = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -6.0, -0.5, 0.0, 1.0, 1.0, 2.0,
                         4.0, 4.0])
    assert torch.equal(deq[0], want)
    lo, hi = codes[0] & 15, codes[0] >> 4
    assert lo.tolist() == [0, 2, 4, 6, 15, 0, 2, 6] and hi.tolist() == [1, 3, 5, 7, 9, 2, 4, 6]


def test_fp4_cache_cpu_roundtrip():
    T, Hkv, D, bs, nb = 9, 2, 32, 4, 4
    g = torch.Generator().manual_seed(0)
    k = torch.randn(T, Hkv * D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv * D, generator=g).to(torch.bfloat16)
    slots = torch.randperm(nb * bs, generator=g)[:T]
    mk = lambda last: torch.zeros(nb, Hkv, bs, last, dtype=torch.uint8)
    kc, vc, ks, vs = mk(D // 2), mk(D // 2), mk(D // 16), mk(D // 16)
    ops.kv_write_fp4(k, v, slots, kc, vc, ks, vs, Hkv, D)
    back = ops.kv_read_fp4(kc, ks, slots, Hkv, D)
    _, _, deq = ref.quantize_nvfp4(k.view(T, Hkv, D))
    assert torch.allclose(back.float(), deq.reshape(T, Hkv * D).to(torch.bfloat16).float())
    err = (back.float() - k.float()).abs().max()
    assert float(err) < 0.6


def test_bulk_write_cpu_matches_per_layer():
    T, L, Hkv, D, bs, nb = 6, 3, 2, 16, 4, 3
    g = torch.Generator().manual_seed(1)
    kv_all = torch.randn(T, L * 2 * Hkv * D, generator=g).to(torch.bfloat16)
    pos = torch.arange(T)
    slots = torch.tensor([0, 5, -1, 7, 2, 11])
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    mk = lambda: [torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16) for _ in range(L)]
    kc, vc, kc2, vc2 = mk(), mk(), mk(), mk()
    ops.kv_bulk_write(kv_all, pos, slots, inv_freq, kc, vc, Hkv, D)
    w = 2 * Hkv * D
    for j in range(L):
        ops.rope_cache(kv_all[:, j * w:(j + 1) * w].clone(), pos, slots, inv_freq, kc2[j], vc2[j],
                       0, Hkv, D)
        assert torch.equal(kc[j], kc2[j]) and torch.equal(vc[j], vc2[j])


def test_tiled_fp8_weight_storage_is_the_same_matrix():
    """Codes stored as [N/16, K/128, 16, 128] tiles stand for the same matrix as row-major
    codes: dequantisation, shard views on tile boundaries, the linear oracle and in-place
    re-quantisation all agree; a slice that cuts a tile is refused."""
    import pytest
    import torch
    from arcticinference_b200.models import quant
    w = (torch.randn(512, 1024) * 0.05).to(torch.bfloat16)
    a = quant.quantize_weight_fp8_row(w, tiled=False)
    b = quant.quantize_weight_fp8_row(w, tiled=True)
    assert tuple(b.shape) == tuple(a.shape) == (512, 1024) and b.q.dim() == 4
    assert torch.equal(b.codes().view(torch.uint8), a.q.view(torch.uint8))
    s, r = b[128:384, 256:768], a[128:384, 256:768]
    assert tuple(s.shape) == (256, 512) and torch.equal(s.scale, r.scale)
    assert torch.equal(s.dequantize(), r.dequantize())
    x = torch.randn(5, 512).to(torch.bfloat16)
    assert torch.equal(quant.linear_fp8_row_ref(x, s), quant.linear_fp8_row_ref(x, r))
    ptr = b.q.data_ptr()
    b.requantize_from(w * 2)
    a.requantize_from(w * 2)
    assert b.q.data_ptr() == ptr and torch.equal(b.dequantize(), a.dequantize())
    with pytest.raises(ValueError):
        b[8:24]
