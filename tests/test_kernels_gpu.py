"""Numerics of the sm_100a kernels against plain PyTorch fp32 restatements."""

import math

import pytest
import torch

from arcticinference_b200 import ops
from arcticinference_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _close(a, b, atol, rtol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), "max err %.4g at %d elements (max ref %.4g)" % (
        float(err.max()), int(bad.sum()), float(b.abs().max()))


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("T,H", [(1, 64), (7, 768), (3, 2048), (33, 4096), (5, 8192)])
def test_rmsnorm(T, H):
    x, w = _rand(T, H), _rand(H)
    y = ops.rmsnorm(x, w, 1e-5)
    _close(y, ref.rmsnorm(x, w, 1e-5), 2e-2, 2e-2)
    res = _rand(T, H)
    res_ref = res.clone()
    y = ops.rmsnorm(x, w, 1e-5, residual=res)
    y_ref = ref.rmsnorm(x, w, 1e-5, residual=res_ref)
    _close(res, res_ref, 1e-2, 1e-2)
    _close(y, y_ref, 3e-2, 2e-2)
    ops.check_status()


def test_rmsnorm_strided_input():
    buf = _rand(9, 3 * 1024)
    x = buf[:, 1024:2048]
    w = _rand(1024)
    _close(ops.rmsnorm(x, w, 1e-6), ref.rmsnorm(x, w, 1e-6), 2e-2, 2e-2)


@pytest.mark.parametrize("T,H", [(3, 768), (17, 1024)])
def test_layernorm(T, H):
    x, r, g, b = _rand(T, H), _rand(T, H), _rand(H), _rand(H)
    _close(ops.layernorm(x, g, b, 1e-12), ref.layernorm(x, g, b, 1e-12), 3e-2, 2e-2)
    _close(ops.layernorm(x, g, b, 1e-12, residual=r), ref.layernorm(x, g, b, 1e-12, residual=r),
           3e-2, 2e-2)


def test_silu_mul():
    x = _rand(19, 2 * 14336)
    _close(ops.silu_mul(x), ref.silu_mul(x), 2e-2, 2e-2)


def test_silu_mul_many_rows_rank_major_blocks():
    # more vectors than one pass of the grid covers; two (gate | up) blocks per row
    T, inter, nblk = 6000, 1792, 2
    x = _rand(T, nblk * 2 * inter)
    got = ops.silu_mul_blocked(x, nblk)
    xb = x.view(T, nblk, 2 * inter)
    exp = torch.cat([ref.silu_mul(xb[:, b]) for b in range(nblk)], dim=1)
    _close(got, exp, 2e-2, 2e-2)


def test_embedding_and_gather():
    table = _rand(1000, 512)
    ids = torch.randint(0, 1000, (37,), device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids])
    # vocab-parallel shard: ids outside [start, start+V) give zeros
    out = ops.embedding(ids + 500, table, vocab_start=600)
    exp = ref.embedding(ids + 500, table, vocab_start=600)
    assert torch.equal(out, exp)
    idx = torch.tensor([5, 0, 36, 7], device=DEV)
    src = _rand(37, 256)
    assert torch.equal(ops.gather_rows(src, idx), src[idx])


def test_argmax_sample():
    logits = _rand(9, 128256, scale=3.0)
    ids, vals = ops.argmax_sample(logits)
    assert torch.equal(ids, logits.float().argmax(-1))
    _close(vals, logits.float().max(-1).values, 1e-6, 0)
    lf = logits.float()
    ids2, _ = ops.argmax_sample(lf, index_offset=1000)
    assert torch.equal(ids2, lf.argmax(-1) + 1000)
    # sampling: distribution sanity on a tiny vocabulary
    small = torch.tensor([[0.0, 1.0, 2.0, -20.0]], device=DEV).repeat(4000, 1)
    temp = torch.ones(4000, device=DEV)
    seeds = torch.arange(4000, device=DEV, dtype=torch.int64) * 7919 + 13
    s_ids, _ = ops.argmax_sample(small, temperature=temp, seeds=seeds)
    freq = torch.bincount(s_ids, minlength=4).float() / 4000
    exp = torch.softmax(small[0], -1)
    assert float((freq - exp).abs().max()) < 0.04
    # a row's draw depends on its logits and seed only, not on where it sits in the batch
    lg = _rand(64, 5000, scale=2.0)
    sd = torch.arange(64, device=DEV, dtype=torch.int64) * 104729 + 7
    tt = torch.full((64,), 0.8, device=DEV)
    base, _ = ops.argmax_sample(lg, temperature=tt, seeds=sd)
    perm = torch.randperm(64, device=DEV)
    moved, _ = ops.argmax_sample(lg[perm].contiguous(), temperature=tt, seeds=sd[perm].contiguous())
    assert torch.equal(moved, base[perm])
    # shards of a split vocabulary: the arg-max over the shards' winners is the full draw
    lo, _ = ops.argmax_sample(lg[:, :2504].contiguous(), temperature=tt, seeds=sd)
    hi, _ = ops.argmax_sample(lg[:, 2504:].contiguous(), temperature=tt, seeds=sd, index_offset=2504)
    assert bool(((base == lo) | (base == hi)).all())


def test_rope_cache():
    T, Hq, Hkv, D, bs, nb = 23, 8, 2, 128, 32, 6
    qkv = _rand(T, (Hq + 2 * Hkv) * D)
    qkv_ref = qkv.clone()
    pos = torch.randint(0, 100000, (T,), device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[3] = -1
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    kc, vc = torch.zeros(nb, Hkv, bs, D, device=DEV, dtype=torch.bfloat16), \
        torch.zeros(nb, Hkv, bs, D, device=DEV, dtype=torch.bfloat16)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    ops.rope_cache(qkv, pos, slots, inv_freq, kc, vc, Hq, Hkv, D)
    ref.rope_cache(qkv_ref, pos, slots, inv_freq, kc_ref, vc_ref, Hq, Hkv, D)
    ops.check_status()
    _close(qkv[:, :Hq * D], qkv_ref[:, :Hq * D], 3e-2, 2e-2)
    _close(kc, kc_ref, 3e-2, 2e-2)
    assert torch.equal(vc, vc_ref)


@pytest.mark.parametrize("fp8", [False, True])
def test_kv_bulk_write(fp8):
    T, L, Hkv, D, bs, nb = 37, 5, 2, 128, 32, 8
    kv_all = _rand(T, L * 2 * Hkv * D)
    pos = torch.randint(0, 100000, (T,), device=DEV)
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[5] = -1
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2, device=DEV).float() / D))
    dt = torch.float8_e4m3fn if fp8 else torch.bfloat16
    mk = lambda: [torch.zeros(nb, Hkv, bs, D, device=DEV, dtype=torch.bfloat16).to(dt) for _ in range(L)]
    kc, vc, kc_ref, vc_ref = mk(), mk(), mk(), mk()
    ks = torch.linspace(0.01, 0.02, L, device=DEV) if fp8 else None
    vs = torch.linspace(0.02, 0.01, L, device=DEV) if fp8 else None
    ops.kv_bulk_write(kv_all, pos, slots, inv_freq, kc, vc, Hkv, D, k_scales=ks, v_scales=vs)
    ops.check_status()
    ref.kv_bulk_write(kv_all, pos, slots, inv_freq, kc_ref, vc_ref, Hkv, D, ks, vs)
    for j in range(L):
        if fp8:
            # one e4m3 step (1/8 relative) where the rotated value sits on a rounding boundary
            _close(kc[j].float() * ks[j], kc_ref[j].float() * ks[j], 3e-2, 0.13)
            assert float((kc[j].float() != kc_ref[j].float()).float().mean()) < 0.02
            assert torch.equal(vc[j].view(torch.uint8), vc_ref[j].view(torch.uint8))
        else:
            _close(kc[j], kc_ref[j], 3e-2, 2e-2)
            assert torch.equal(vc[j], vc_ref[j])


def test_kv_fp4_write_and_read():
    T, Hkv, D, bs, nb = 29, 4, 128, 16, 4
    k, v = _rand(T, Hkv * D), _rand(T, Hkv * D, scale=3.0)
    k[2, :16] = 0                      # an all-zero group
    slots = torch.randperm(nb * bs, device=DEV)[:T]
    slots[7] = -1
    mk = lambda last: torch.zeros(nb, Hkv, bs, last, device=DEV, dtype=torch.uint8)
    kc, vc, ksc, vsc = mk(D // 2), mk(D // 2), mk(D // 16), mk(D // 16)
    ops.kv_write_fp4(k, v, slots, kc, vc, ksc, vsc, Hkv, D)
    ops.check_status()
    ok = slots >= 0
    blk, off = slots[ok] // bs, slots[ok] % bs
    for src, codes, scales in ((k, kc, ksc), (v, vc, vsc)):
        rc, rs, deq = ref.quantize_nvfp4(src.view(T, Hkv, D))
        assert torch.equal(scales[blk, :, off], rs[ok])
        got = codes[blk, :, off]
        # identical codes except where a scaled value sits exactly between two e2m1 values
        assert float((got != rc[ok]).float().mean()) < 0.005
        back = ops.kv_read_fp4(codes, scales, slots[ok], Hkv, D).view(-1, Hkv, D)
        # the error of one element is at most half an e2m1 step (1 at the top) times the scale
        bound = rs[ok].view(torch.float8_e4m3fn).float().repeat_interleave(16, -1) * 1.0 + 1e-3
        assert bool(((back.float() - src.view(T, Hkv, D)[ok].float()).abs() <= bound * 1.01).all())
        same = got == rc[ok]
        both = same.repeat_interleave(2, -1)
        _close(back.float()[both], deq[ok][both], 1e-2, 1e-2)
    assert int(kc[slots[7] // bs if slots[7] >= 0 else 0].sum()) >= 0   # padding token wrote nothing
    ops.check_status()


# ------------------------------------------------------------------------------------ GEMM
GEMM_SHAPES = [
    (128, 128, 64), (128, 256, 128), (300, 512, 256), (1000, 1024, 4096), (4096, 6144, 4096),
    (2048, 4096, 14336), (257, 136, 72), (513, 128256, 512),
    # feature-major (decode) orientation
    (1, 4096, 4096), (8, 6144, 4096), (17, 4096, 14336), (64, 28672, 4096), (130, 1024, 512),
    (256, 4096, 4096), (3, 136, 72),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_linear(M, N, K):
    x = _rand(M, K)
    w = _rand(N, K, scale=1.0 / math.sqrt(K))
    y = ops.linear(x, w)
    ops.check_status()
    _close(y, ref.linear(x, w), 3e-2, 2e-2)


@pytest.mark.parametrize("M", [5, 128, 700])
def test_linear_epilogue(M):
    N, K = 768, 3072
    x, w = _rand(M, K), _rand(N, K, scale=1.0 / math.sqrt(K))
    b, r = _rand(N), _rand(M, N)
    _close(ops.linear(x, w, bias=b), ref.linear(x, w, bias=b), 3e-2, 2e-2)
    _close(ops.linear(x, w, bias=b, act="gelu"), ref.linear(x, w, bias=b, act="gelu"), 3e-2, 2e-2)
    _close(ops.linear(x, w, bias=b, residual=r), ref.linear(x, w, bias=b, residual=r), 4e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_linear_split_k(splits):
    M, N, K = 24, 1024, 4096
    x, w = _rand(M, K), _rand(N, K, scale=1.0 / math.sqrt(K))
    b, r = _rand(N), _rand(M, N)
    y = ops.linear(x, w, bias=b, residual=r, force_splits=splits)
    ops.check_status()
    _close(y, ref.linear(x, w, bias=b, residual=r), 4e-2, 2e-2)


def test_linear_strided_views():
    # x is a column slice of a wider buffer; out is a column slice too
    buf = _rand(200, 3 * 512)
    w = _rand(384, 512, scale=1.0 / math.sqrt(512))
    out_buf = torch.zeros(200, 1024, device=DEV, dtype=torch.bfloat16)
    ops.linear(buf[:, 512:1024], w, out=out_buf[:, 128:512])
    ops.check_status()
    _close(out_buf[:, 128:512], ref.linear(buf[:, 512:1024], w), 3e-2, 2e-2)
    assert float(out_buf[:, :128].abs().max()) == 0 and float(out_buf[:, 512:].abs().max()) == 0


@pytest.mark.parametrize("M,blk,K", [(300, 192, 512), (64, 192, 512), (1000, 80, 512),
                                     (64, 192, 4096), (128, 512, 2048), (5, 128, 8192)])
def test_linear_scatter_epilogue_local_destinations(M, blk, K):
    """The scatter epilogue with both destinations in this GPU's memory: feature block j of
    token m must land in buffer j at row m + offset (blk=192 takes the coalesced store path,
    blk=80 the direct one; with at most 128 tokens and a long K the CTAs of a cluster split K
    and the CTA that finishes a column range stores it to its owner)."""
    import ctypes
    from arcticinference_b200.ops import native
    world, off = 2, 7
    x = _rand(M, K)
    w = _rand(world * blk, K, scale=1.0 / math.sqrt(K))
    bufs = [torch.zeros(M + 2 * off, blk, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    native.declare("ab200_linear_bf16_scatter", I, [P, LL, P, LL, P, I, I, LL, LL, I, I, I, P, P])
    rc = native.lib().ab200_linear_bf16_scatter(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), ptrs, world, blk, off, blk, M,
        world * blk, K, native.status_buffer(x.device).data_ptr(), native.stream_ptr())
    assert rc == 0
    ops.check_status()
    want = ref.linear(x, w)
    for j, b in enumerate(bufs):
        _close(b[off:off + M], want[:, j * blk:(j + 1) * blk], 3e-2, 2e-2)
        assert float(b[:off].abs().max()) == 0 and float(b[off + M:].abs().max()) == 0


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 256, 512), (1024, 192, 128)])
def test_gemm_nn(M, N, K):
    x, wt = _rand(M, K), _rand(K, N, scale=1.0 / math.sqrt(K))
    y = ops.gemm_nn(x, wt)
    ops.check_status()
    _close(y, x.float() @ wt.float(), 3e-2, 2e-2)


# ------------------------------------------------------------------------------- attention
def _paged_case(q_lens, kv_lens, Hq, Hkv, D, bs, seed=0):
    torch.manual_seed(seed)
    T = sum(q_lens)
    nblk_seq = [(k + bs - 1) // bs for k in kv_lens]
    nb = sum(nblk_seq) + 3
    perm = torch.randperm(nb)[: sum(nblk_seq)].int()
    maxb = max(nblk_seq)
    bt = torch.zeros(len(q_lens), maxb, dtype=torch.int32)
    o = 0
    for i, n in enumerate(nblk_seq):
        bt[i, :n] = perm[o:o + n]
        o += n
    q = _rand(T, Hq * D)
    kc = _rand(nb, Hkv, bs, D)
    vc = _rand(nb, Hkv, bs, D)
    return q, kc, vc, bt.to(DEV)


@pytest.mark.parametrize("q_lens,kv_lens,Hq,Hkv,D,bs", [
    ([128], [128], 4, 1, 128, 32),
    ([200, 57], [200, 57], 8, 2, 128, 16),
    ([300], [812], 8, 2, 128, 64),           # chunked prefill with a cached prefix
    ([1, 1, 1], [700, 33, 129], 8, 2, 128, 32),   # decode
    ([4, 4], [1500, 260], 32, 8, 128, 32),   # speculative verification, 4 tokens per sequence
    ([100, 30], [100, 30], 16, 2, 128, 128),  # G = 8
    ([64, 200], [64, 200], 12, 12, 64, 16),  # head_dim 64, no GQA
])
def test_paged_attention(q_lens, kv_lens, Hq, Hkv, D, bs):
    q, kc, vc, bt = _paged_case(q_lens, kv_lens, Hq, Hkv, D, bs)
    meta = ops.build_attention_metadata(q_lens, kv_lens, bt, Hq // Hkv, Hq, D, DEV)
    lse = torch.empty(sum(q_lens), Hq, device=DEV, dtype=torch.float32)
    out = ops.attention(q, kc, vc, meta, Hq, Hkv, D, lse_out=lse)
    ops.check_status()
    exp, lse_ref = ref.attention(q, kc, vc, bt, q_lens, kv_lens, Hq, Hkv, D, 1 / math.sqrt(D),
                                 return_lse=True)
    _close(out, exp, 2e-2, 2e-2)
    _close(lse, lse_ref, 2e-2, 1e-2)


def test_paged_attention_split_kv():
    q_lens, kv_lens, Hq, Hkv, D, bs = [1, 2], [4000, 1111], 8, 2, 128, 32
    q, kc, vc, bt = _paged_case(q_lens, kv_lens, Hq, Hkv, D, bs)
    meta = ops.build_attention_metadata(q_lens, kv_lens, bt, Hq // Hkv, Hq, D, DEV)
    assert meta.max_splits > 1
    out = ops.attention(q, kc, vc, meta, Hq, Hkv, D)
    ops.check_status()
    exp = ref.attention(q, kc, vc, bt, q_lens, kv_lens, Hq, Hkv, D, 1 / math.sqrt(D))
    _close(out, exp, 2e-2, 2e-2)


@pytest.mark.parametrize("H,D,seq_lens", [(12, 64, [50, 128, 3, 512]), (4, 128, [77, 300])])
def test_encoder_attention(H, D, seq_lens):
    T = sum(seq_lens)
    qkv = _rand(T, 3 * H * D)
    q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
    out = ops.attention_contiguous(q, k, v, seq_lens, H, D)
    ops.check_status()
    _close(out, ref.attention_contiguous(q, k, v, seq_lens, H, D, 1 / math.sqrt(D)), 2e-2, 2e-2)


# ------------------------------------------------------------------------------ speculator
from arcticinference_b200.ops import spec_ops  # noqa: E402


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (37, 4096), (5, 1000), (3, 8192)])
def test_spec_ln(rows, hidden):
    x, w, b = _rand(rows, hidden), _rand(hidden), _rand(hidden)
    _close(spec_ops.spec_ln(x, w, b), spec_ops.spec_ln_ref(x, w, b), 3e-2, 2e-2)
    _close(spec_ops.spec_ln(x, None, None, 1e-6, 0.7071), spec_ops.spec_ln_ref(x, None, None, 1e-6, 0.7071),
           2e-2, 2e-2)
    buf = _rand(rows, 2 * hidden)   # pitched rows
    _close(spec_ops.spec_ln(buf[:, hidden:], w, None), spec_ops.spec_ln_ref(buf[:, hidden:], w, None),
           3e-2, 2e-2)


@pytest.mark.parametrize("B,D", [(1, 4096), (33, 4096), (4, 1024), (7, 520)])
@pytest.mark.parametrize("tanh", [False, True])
def test_sum_lstm(B, D, tanh):
    gates, prev_c = _rand(B, 4 * D), _rand(B, D)
    emb = _rand(100, D)
    tok = torch.randint(0, 100, (B,), device=DEV)
    wc, bc, ws, bs = _rand(D), _rand(D, scale=0.1), _rand(D), _rand(D, scale=0.1)
    for pc in (None, prev_c):
        c, h = spec_ops.sum_lstm(gates, emb, tok, 1.3, pc, wc, bc, ws, bs, 1e-6, tanh)
        c_ref, h_ref = spec_ops.sum_lstm_ref(gates, emb, tok, 1.3, pc, wc, bc, ws, bs, 1e-6, tanh)
        _close(c, c_ref, 4e-2, 3e-2)
        _close(h, h_ref, 6e-2, 3e-2)
    emb4 = _rand(100, 4 * D)        # untied gate embeddings
    c, h = spec_ops.sum_lstm(gates, emb4, tok, 0.9, prev_c, wc, None, ws, None)
    c_ref, h_ref = spec_ops.sum_lstm_ref(gates, emb4, tok, 0.9, prev_c, wc, None, ws, None)
    _close(c, c_ref, 4e-2, 3e-2)
    _close(h, h_ref, 6e-2, 3e-2)


def test_mlp_spec_step():
    B, D = 19, 4096
    proj, emb = _rand(B, D), _rand(50, D)
    tok = torch.randint(0, 50, (B,), device=DEV)
    w, b = _rand(D), _rand(D, scale=0.1)
    _close(spec_ops.mlp_spec_step(proj, emb, tok, 2.1, w, b),
           spec_ops.mlp_spec_step_ref(proj, emb, tok, 2.1, w, b), 5e-2, 3e-2)


def test_verify_greedy():
    input_ids = torch.tensor([10, 11, 12, 13, 20, 30, 31, 32], device=DEV)
    target = torch.tensor([11, 12, 99, 14, 21, 31, 32, 33], device=DEV)
    row_start = torch.tensor([0, 4, 5, -1], dtype=torch.int32, device=DEV)
    num_draft = torch.tensor([3, 0, 2, 0], dtype=torch.int32, device=DEV)
    acc, nxt, sel, out = spec_ops.verify_greedy(input_ids, target, row_start, num_draft, 3)
    assert acc.tolist() == [2, 0, 2, 0]
    assert nxt.tolist()[:3] == [99, 21, 33]
    assert sel.tolist()[:3] == [2, 4, 7]
    assert out.tolist()[:3] == [[11, 12, 99, -1], [21, -1, -1, -1], [31, 32, 33, -1]]
    assert out.tolist()[3] == [-1, -1, -1, -1]


# ------------------------------------------------------------------------------------- fp8
from arcticinference_b200.models import quant  # noqa: E402


def test_quant_fp8_matches_reference():
    x = _rand(37, 1024, scale=2.0)
    xq, sx = ops.quant_fp8(x)
    rq, rs = quant.quant_activation_ref(x)
    _close(sx, rs, 1e-7, 1e-5)
    # codes may differ by one ulp where the scaled value sits on a rounding boundary
    diff = (xq.float() - rq.float()).abs()
    assert float((diff > 0).float().mean()) < 0.01
    back = xq.float().view(37, 8, 128) * sx.t().unsqueeze(-1)
    _close(back.view(37, 1024), x, 0.05 * float(x.float().abs().max()), 0.07)


def _w8a8_ref(x, w):
    """fp32 product of the activations as the quantisation kernel coded them (that kernel has
    its own test) and the de-quantised weight: a code that sits on a rounding boundary must not
    decide the GEMM test."""
    xq, sx_t = ops.quant_fp8(x)
    M, K = x.shape
    xd = xq.float().view(M, K // 128, 128) * sx_t[:, :M].t().unsqueeze(-1)
    return xd.view(M, K) @ w.dequantize().float().t()


@pytest.mark.parametrize("M,N,K", [
    (8, 4096, 4096), (32, 6144, 4096), (100, 1024, 512), (128, 4096, 14336), (1, 256, 128),
    (129, 256, 256), (512, 1024, 1024), (2048, 6144, 4096), (1000, 28672, 4096), (300, 384, 1792),
])
def test_linear_fp8(M, N, K):
    x = _rand(M, K)
    w = quant.quantize_weight_fp8(_rand(N, K, scale=1.0 / math.sqrt(K)))
    # W8A8 kernel; oracle: the same quantised operands multiplied in fp32
    y = ops.linear_fp8(x, w, mode="w8a8")
    ops.check_status()
    _close(y, _w8a8_ref(x, w), 5e-2, 2e-2)
    # default dispatch (weight-only fp8 for few tokens, expanded bf16 for long prefill);
    # oracle: bf16 activations times the de-quantised weight
    y2 = ops.linear(x, w)
    ops.check_status()
    if M <= ops.W8A16_MAX_TOKENS or M >= ops.DEQUANT_MIN_TOKENS:
        _close(y2, ref.linear(x, w.dequantize()), 5e-2, 2e-2)
    else:   # in between, activations are quantised too
        _close(y2, _w8a8_ref(x, w), 5e-2, 2e-2)


@pytest.mark.parametrize("splits", [1, 2, 4])
def test_linear_w8a16_split_k(splits):
    x = _rand(24, 4096)
    w = quant.quantize_weight_fp8(_rand(1024, 4096, scale=1.0 / 64))
    y = ops.linear_fp8(x, w, force_splits=splits)
    ops.check_status()
    _close(y, ref.linear(x, w.dequantize()), 5e-2, 2e-2)


def test_linear_fp8_shard_views():
    x = _rand(64, 1024)
    w = quant.quantize_weight_fp8(_rand(2048, 2048, scale=0.03))
    xk = _rand(64, 2048)
    rows = w[512:1024]
    _close(ops.linear(xk, rows), ref.linear(xk, rows.dequantize()), 5e-2, 2e-2)
    cols = w[:, 1024:2048]
    xs = xk[:, 1024:2048]          # strided activation view, K-slice of the weight
    _close(ops.linear(xs, cols), ref.linear(xs, cols.dequantize()), 5e-2, 2e-2)
    _close(ops.linear(x, w[256:768, :1024]), ref.linear(x, w[256:768, :1024].dequantize()), 5e-2, 2e-2)
    big = _rand(300, 1024)
    _close(ops.linear_fp8(big, w[256:768, :1024], mode="w8a8"),
           _w8a8_ref(big, w[256:768, :1024]), 5e-2, 2e-2)
    ops.check_status()


# ------------------------------------------- fp8 with per-token / per-feature scales (W8A8)
def _row_ref(xq, w, **kw):
    """fp32 product of the codes the quantiser produced (it has its own test) and the weight's
    codes, scaled per token and per feature."""
    return quant.linear_fp8_row_ref(xq, w, **kw)


@pytest.mark.parametrize("M,K", [(1, 64), (37, 1024), (5, 4096), (3, 14336), (2, 28672), (9, 136)])
def test_quant_fp8_row_matches_reference(M, K):
    x = _rand(M, K, scale=2.0)
    got = ops.quant_fp8_row(x)
    want = quant.quant_activation_row_ref(x)
    _close(got.scale, want.scale, 1e-9, 1e-6)
    diff = (got.q.float() - want.q.float()).abs()
    assert float((diff > 0).float().mean()) < 0.01
    _close(got.dequantize(), x, 0.04 * float(x.float().abs().max()), 0.07)


@pytest.mark.parametrize("T,H,res", [(33, 4096, True), (5, 8192, True), (7, 768, False),
                                     (3, 2048, True), (2, 5120, True), (1, 64, False)])
def test_rmsnorm_quant_matches_unfused(T, H, res):
    x, w = _rand(T, H), _rand(H, scale=0.5) + 1.0
    r1 = _rand(T, H) if res else None
    r2 = r1.clone() if res else None
    got = ops.rmsnorm(x, w, 1e-5, residual=r1, quant=True)
    y = ops.rmsnorm(x, w, 1e-5, residual=r2)
    want = ops.quant_fp8_row(y)
    ops.check_status()
    if res:
        assert torch.equal(r1, r2)
    _close(got.scale, want.scale, 1e-9, 1e-6)
    assert torch.equal(got.q.view(torch.uint8), want.q.view(torch.uint8))


@pytest.mark.parametrize("T,inter,nblk", [(9, 14336, 1), (4, 1792, 8), (3, 28672, 1), (5, 256, 2),
                                          (2, 3584, 8)])
def test_silu_mul_quant_matches_unfused(T, inter, nblk):
    x = _rand(T, nblk * 2 * inter)
    got = ops.silu_mul_blocked(x, nblk, quant=True)
    want = ops.quant_fp8_row(ops.silu_mul_blocked(x, nblk))
    ops.check_status()
    _close(got.scale, want.scale, 1e-9, 1e-6)
    assert torch.equal(got.q.view(torch.uint8), want.q.view(torch.uint8))


@pytest.mark.parametrize("M,N,K", [
    (8, 4096, 4096), (32, 6144, 4096), (100, 1024, 512), (128, 4096, 14336), (1, 256, 128),
    (129, 256, 256), (200, 4096, 4096), (512, 1024, 1024), (2048, 6144, 4096),
    (1000, 28672, 4096), (300, 384, 1792), (700, 136, 80), (17, 4096, 14336),
])
def test_linear_fp8_row(M, N, K):
    x = _rand(M, K)
    w = quant.quantize_weight_fp8_row(_rand(N, K, scale=1.0 / math.sqrt(K)))
    xq = ops.quant_fp8_row(x)
    y = ops.linear(xq, w)
    ops.check_status()
    _close(y, _row_ref(xq, w), 3e-2, 2e-2)
    # bf16 activations are quantised on the way in; against the unquantised product the error
    # is the e4m3 rounding of the activations (up to 2^-4 relative per element, i.e. a few
    # hundredths of the output's standard deviation, 1 here; the extremes over a million
    # outputs reach 0.15)
    y2 = ops.linear(x, w)
    ops.check_status()
    assert torch.equal(y, y2)
    _close(y2, ref.linear(x, w.dequantize()), 0.25, 5e-2)


@pytest.mark.parametrize("M", [5, 128, 200, 700])
def test_linear_fp8_row_epilogue(M):
    N, K = 768, 3072
    xq = ops.quant_fp8_row(_rand(M, K))
    w = quant.quantize_weight_fp8_row(_rand(N, K, scale=1.0 / math.sqrt(K)))
    b, r = _rand(N), _rand(M, N)
    _close(ops.linear(xq, w, bias=b), _row_ref(xq, w, bias=b), 3e-2, 2e-2)
    _close(ops.linear(xq, w, bias=b, act="gelu"), _row_ref(xq, w, bias=b, act="gelu"), 3e-2, 2e-2)
    _close(ops.linear(xq, w, bias=b, residual=r), _row_ref(xq, w, bias=b, residual=r), 4e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 4096, 4096), (64, 6144, 4096), (128, 4096, 14336),
                                   (3, 512, 1024), (128, 1000, 2048), (96, 4096, 512)])
def test_linear_one_row_of_tiles_splits_k_inside_clusters(M, N, K):
    """At most 128 tokens and few output tiles: the K range is split over the CTAs of a
    thread-block cluster, which add their partial sums through shared memory. The result
    matches the fp32 reference, does not depend on timing, and is the same whether or not
    the weight was declared a parameter (its first tiles are then requested early)."""
    x = _rand(M, K)
    wf = _rand(N, K, scale=1.0 / math.sqrt(K))
    b, r = _rand(N), _rand(M, N)
    # bf16 operands
    y = ops.linear(x, wf, bias=b, residual=r)
    ops.check_status()
    _close(y, ref.linear(x, wf, b, r), 3e-2, 2e-2)
    assert torch.equal(y, ops.linear(x, wf, bias=b, residual=r))
    ops.mark_static(wf)
    assert torch.equal(y, ops.linear(x, wf, bias=b, residual=r))
    # e4m3 operands
    w = quant.quantize_weight_fp8_row(wf)
    xq = ops.quant_fp8_row(x)
    yq = ops.linear(xq, w, residual=r)
    ops.check_status()
    _close(yq, _row_ref(xq, w, residual=r), 4e-2, 2e-2)
    ops.mark_static(w)
    assert torch.equal(yq, ops.linear(xq, w, residual=r))
    ops.clear_static()
    ops.check_status()


@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_linear_fp8_row_split_k(splits):
    M, N, K = 24, 1024, 4096
    xq = ops.quant_fp8_row(_rand(M, K))
    w = quant.quantize_weight_fp8_row(_rand(N, K, scale=1.0 / math.sqrt(K)))
    y = ops.linear(xq, w, force_splits=splits)
    ops.check_status()
    _close(y, _row_ref(xq, w), 3e-2, 2e-2)


@pytest.mark.parametrize("M,N,K", [(128, 4096, 4096), (24, 1024, 512), (700, 2048, 1024), (200, 512, 256)])
def test_linear_fp8_row_tiled_storage(M, N, K):
    """The optional 16-row x 128-byte tile storage of the codes gives the same product, also
    through shard views on tile boundaries."""
    wf = _rand(N, K, scale=1.0 / math.sqrt(K))
    xq = ops.quant_fp8_row(_rand(M, K))
    flat, tiled = quant.quantize_weight_fp8_row(wf), quant.quantize_weight_fp8_row(wf, tiled=True)
    assert not flat.tiled and tiled.tiled
    y = ops.linear(xq, flat)
    assert torch.equal(ops.linear(xq, tiled), y)
    assert torch.equal(ops.linear(xq, tiled[N // 4:N // 2]), ops.linear(xq, flat[N // 4:N // 2]))
    xs = ops.quant_fp8_row(_rand(M, K // 2))
    assert torch.equal(ops.linear(xs, tiled[:, K // 2:]), ops.linear(xs, flat[:, K // 2:]))
    ops.check_status()


def test_linear_fp8_row_shard_views():
    w = quant.quantize_weight_fp8_row(_rand(2048, 2048, scale=0.03))
    xk = ops.quant_fp8_row(_rand(64, 2048))
    rows = w[512:1024]
    _close(ops.linear(xk, rows), _row_ref(xk, rows), 3e-2, 2e-2)
    cols = w[:, 1024:2048]          # K shard: strided weight view, all feature scales
    xs = ops.quant_fp8_row(_rand(300, 1024))
    _close(ops.linear(xs, cols), _row_ref(xs, cols), 3e-2, 2e-2)
    _close(ops.linear(xs, w[256:768, :1024]), _row_ref(xs, w[256:768, :1024]), 3e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("M,blk,K,rank", [(300, 192, 512, 1), (64, 192, 4096, 1), (128, 512, 4096, 2),
                                          (2000, 256, 1024, 3)])
def test_linear_fp8_row_scatter_walks_tiles_from_its_own_rank(M, blk, K, rank):
    """With a completion signal attached the scatter GEMM knows its rank and starts its walk
    over the output tiles at its own share of the columns (so that ranks store into different
    destinations at any moment). Same result; the signal reaches every rank's flag word."""
    import ctypes
    from arcticinference_b200.ops import native
    world, off = 4, 3
    xq = ops.quant_fp8_row(_rand(M, K))
    w = quant.quantize_weight_fp8_row(_rand(world * blk, K, scale=1.0 / math.sqrt(K)))
    bufs = [torch.zeros(M + 2 * off, blk, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    chan = torch.zeros(world, 64, device=DEV, dtype=torch.int32)   # per "rank": flags | done | epoch
    flag_ptrs = (ctypes.c_void_p * world)(*[chan[r].data_ptr() for r in range(world)])
    sync = native.PeerSync()
    sync.sig_flag_ptrs = ctypes.cast(flag_ptrs, ctypes.c_void_p)
    sync.sig_done_ctr = chan[rank].data_ptr() + 128
    sync.sig_epoch_ctr = chan[rank].data_ptr() + 192
    sync.sig_rank, sync.sig_world = rank, world
    ops.linear_fp8_row(xq, w, peer=(ptrs, world, blk, off, blk), sync=sync)
    ops.check_status()
    want = _row_ref(xq, w)
    for j, b in enumerate(bufs):
        _close(b[off:off + M], want[:, j * blk:(j + 1) * blk], 3e-2, 2e-2)
        assert float(b[:off].abs().max()) == 0 and float(b[off + M:].abs().max()) == 0
    c = chan.cpu()
    assert all(int(c[r, rank]) == 1 for r in range(world))     # every rank's word of this sender
    assert int(c[rank, 48]) == 1 and int(c[rank, 32]) == 0      # epoch advanced, counter reset


@pytest.mark.parametrize("M,blk,K", [(300, 192, 512), (64, 192, 512), (1000, 80, 512),
                                     (64, 192, 4096), (128, 512, 4096), (5, 128, 8192)])
def test_linear_fp8_row_scatter_epilogue_local_destinations(M, blk, K):
    import ctypes
    world, off = 2, 7
    xq = ops.quant_fp8_row(_rand(M, K))
    w = quant.quantize_weight_fp8_row(_rand(world * blk, K, scale=1.0 / math.sqrt(K)))
    bufs = [torch.zeros(M + 2 * off, blk, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    ops.linear_fp8_row(xq, w, peer=(ptrs, world, blk, off, blk))
    ops.check_status()
    want = _row_ref(xq, w)
    for j, b in enumerate(bufs):
        _close(b[off:off + M], want[:, j * blk:(j + 1) * blk], 3e-2, 2e-2)
        assert float(b[:off].abs().max()) == 0 and float(b[off + M:].abs().max()) == 0
