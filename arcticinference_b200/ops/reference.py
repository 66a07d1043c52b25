"""Plain PyTorch restatements of every op in :mod:`arcticinference_b200.ops`.

They serve two purposes: they are the fp32 oracles the GPU numerics tests
compare the sm_100a kernels against, and they are the implementation used for
CPU tensors (unit tests of the engine, ``gloo`` multi-process tests). They are
never used for CUDA tensors by the engine.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def linear(x, w, bias=None, residual=None, act=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if act == "gelu":
        y = F.gelu(y)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def embedding(ids, table, vocab_start=0):
    local = ids - vocab_start
    valid = (local >= 0) & (local < table.shape[0])
    out = table[local.clamp(0, table.shape[0] - 1)]
    return out * valid.unsqueeze(-1).to(out.dtype)


def rmsnorm(x, weight, eps, residual=None):
    """Returns y; when ``residual`` is given it is updated in place with x + residual."""
    if residual is not None:
        s = (x.float() + residual.float()).to(x.dtype)
        residual.copy_(s)
        xf = s.float()
    else:
        xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype)


def topk_topp_mask(logits, temperature=None, top_k=None, top_p=None):
    """y = logits / temperature where a token is in the top-k / top-p set, -inf elsewhere. The
    k largest stay; of those a token stays iff the probability mass of the tokens strictly more
    likely than it is at most top_p (of the top-k set's mass). Ties for the k-th place go to
    the lowest token ids; at the top-p cut equal logits stay or go together. logits fp32 [B, V]; temperature fp32 [B]; top_k int64 [B] (<= 0: off); top_p
    fp32 [B] (>= 1: off)."""
    B, V = logits.shape
    x = logits.float()
    if temperature is not None:
        x = x * (1.0 / temperature.float().clamp(min=1e-5)).unsqueeze(1)
    vals, order = x.sort(dim=-1, descending=True, stable=True)   # ties in token-id order
    keep = torch.ones_like(x, dtype=torch.bool)
    in_k_sorted = None
    if top_k is not None:
        k = torch.where((top_k > 0) & (top_k < V), top_k, torch.full_like(top_k, V))
        in_k_sorted = torch.arange(V, device=x.device).unsqueeze(0) < k.unsqueeze(1)
        keep = torch.zeros_like(keep).scatter(1, order, in_k_sorted)
    if top_p is not None:
        m = vals[:, :1]
        w_sorted = torch.exp(vals - m)
        if in_k_sorted is not None:
            w_sorted = w_sorted * in_k_sorted
        z = w_sorted.sum(-1, keepdim=True)
        before = w_sorted.cumsum(-1) - w_sorted          # mass ahead of each sorted position
        # mass strictly above a value: what lies ahead of the first position holding it
        first = torch.searchsorted((-vals).contiguous(), (-x).contiguous(), side="left")
        above = before.gather(1, first.clamp(max=V - 1))
        keep &= (above <= top_p.float().unsqueeze(1) * z) | (top_p.float().unsqueeze(1) >= 1.0)
    return torch.where(keep, x, torch.full_like(x, float("-inf")))


def qk_norm(qkv, wq, wk, Hq, Hkv, D, eps):
    """In place: RMSNorm over head_dim of each of the Hq query and Hkv key heads of every row
    of ``qkv`` [T, (Hq + 2*Hkv) * D]; ``wq`` / ``wk`` [D] are shared by the heads."""
    T = qkv.shape[0]
    for lo, n, w in ((0, Hq, wq), (Hq * D, Hkv, wk)):
        if n == 0:
            continue
        x = qkv[:, lo:lo + n * D].reshape(T, n, D).float()
        inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        qkv[:, lo:lo + n * D] = (x * inv * w.float()).to(qkv.dtype).reshape(T, n * D)
    return qkv


def layernorm(x, gamma, beta, eps, residual=None):
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
    return F.layer_norm(xf, (x.shape[-1],), gamma.float(), beta.float(), eps).to(x.dtype)


def silu_mul(x):
    inter = x.shape[-1] // 2
    g, u = x[..., :inter].float(), x[..., inter:].float()
    return (F.silu(g) * u).to(x.dtype)


def silu_mul_blocked(x, nblk=1):
    T, width = x.shape
    inter = width // (2 * nblk)
    v = x.view(T, nblk, 2, inter).float()
    return (F.silu(v[:, :, 0]) * v[:, :, 1]).reshape(T, nblk * inter).to(x.dtype)


def rope_rotate(x, positions, inv_freq):
    """neox pairing: element i is rotated with element i + D/2. x: [T, H, D]."""
    ang = positions.float().unsqueeze(-1) * inv_freq.float().unsqueeze(0)  # [T, D/2]
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(x.dtype)


def rope_cache(qkv, positions, slots, inv_freq, k_cache, v_cache, Hq, Hkv, D, rotate_q=True):
    """In-place RoPE on q (and k), then write k, v into caches [nb, Hkv, bs, D]."""
    T = qkv.shape[0]
    bs = k_cache.shape[2]
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D: (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D: (Hq + 2 * Hkv) * D].view(T, Hkv, D)
    if rotate_q:
        q.copy_(rope_rotate(q, positions, inv_freq))
    k_rot = rope_rotate(k, positions, inv_freq)
    if slots is not None:
        ok = slots >= 0
        s = slots[ok]
        blk, off = s // bs, s % bs
        k_cache[blk, :, off] = k_rot[ok]
        v_cache[blk, :, off] = v[ok]


def kv_bulk_write(kv_all, positions, slots, inv_freq, k_caches, v_caches, Hkv, D,
                  k_scales=None, v_scales=None):
    """K/V of several layers at once: kv_all [T, L*2*Hkv*D], layer j = [k heads | v heads].
    Caches bf16, or float8_e4m3fn with one scale per layer and tensor."""
    T = kv_all.shape[0]
    width = 2 * Hkv * D
    ok = slots >= 0
    s = slots[ok]
    for j, (kc, vc) in enumerate(zip(k_caches, v_caches)):
        bs = kc.shape[2]
        blk, off = s // bs, s % bs
        k = kv_all[:, j * width: j * width + Hkv * D].reshape(T, Hkv, D)
        v = kv_all[:, j * width + Hkv * D: (j + 1) * width].reshape(T, Hkv, D)
        k_rot = rope_rotate(k, positions, inv_freq)
        if kc.dtype == torch.float8_e4m3fn:
            kq = (k_rot.float() / float(k_scales[j])).clamp(-448, 448).to(torch.float8_e4m3fn)
            vq = (v.float() / float(v_scales[j])).clamp(-448, 448).to(torch.float8_e4m3fn)
            kc.view(torch.uint8)[blk, :, off] = kq[ok].view(torch.uint8)
            vc.view(torch.uint8)[blk, :, off] = vq[ok].view(torch.uint8)
        else:
            kc[blk, :, off] = k_rot[ok]
            vc[blk, :, off] = v[ok]


E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quantize_nvfp4(x: torch.Tensor):
    """[..., D] -> (codes uint8 [..., D/2], scales uint8 (e4m3 bits) [..., D/16], dequantised
    fp32 [..., D]). Groups of 16 share scale = e4m3(amax / 6); elements round to the nearest
    e2m1 value, ties to the even code; even element in the low nibble."""
    D = x.shape[-1]
    g = x.float().reshape(*x.shape[:-1], D // 16, 16)
    amax = g.abs().amax(-1, keepdim=True)
    sb = (amax / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    sd = sb.float()
    y = torch.where(sd > 0, g / sd, torch.zeros_like(g))
    vals = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=x.device)
    a = y.abs().clamp(max=6.0)
    # nearest code, ties to even code index
    d = (a.unsqueeze(-1) - vals).abs()
    best = d.argmin(-1)
    nxt = (best + 1).clamp(max=7)
    tie = (d.gather(-1, nxt.unsqueeze(-1)).squeeze(-1) == d.gather(-1, best.unsqueeze(-1)).squeeze(-1)) \
        & (nxt != best)
    code = torch.where(tie & (best % 2 == 1), nxt, best)
    deq = vals[code] * torch.sign(y) * sd
    code = code | ((y < 0) | ((y == 0) & torch.signbit(y))).long() * 8
    code = code.reshape(*x.shape[:-1], D // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8)
    return packed, sb.view(torch.uint8).reshape(*x.shape[:-1], D // 16), deq.reshape(x.shape)


def bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps):
    x = word[ids].float() + pos[positions].float() + \
        typ[type_ids if type_ids is not None else torch.zeros_like(ids)].float()
    y = torch.nn.functional.layer_norm(x, (x.shape[-1],), gamma.float(), beta.float(), eps)
    return y.to(word.dtype)


def pool_normalize(h, starts, mode="cls", normalize=True):
    """h [T, H]; starts [S+1] row offsets. Returns fp32 [S, H]."""
    out = []
    st = [int(v) for v in starts]
    for i in range(len(st) - 1):
        rows = h[st[i]:st[i + 1]].float()
        if mode == "cls":
            v = rows[0]
        elif mode == "last":
            v = rows[-1]
        else:
            v = rows.mean(0)
        if normalize:
            v = v / v.norm().clamp_min(1e-12)
        out.append(v)
    return torch.stack(out)


def gather_rows(src, idx):
    return src[idx]


def argmax_sample(logits, temperature=None, seeds=None, index_offset=0):
    """Greedy where temperature <= 0; elsewhere one draw per row from softmax(logits / T) with
    a generator seeded by that row's seed, so that a row's token does not depend on which
    other rows share the batch (as with the per-row Gumbel noise of the CUDA kernel)."""
    ids = logits.float().argmax(-1)
    vals = logits.float().max(-1).values
    if temperature is not None and bool((temperature > 0).any()):
        t = temperature.clamp_min(1e-6).unsqueeze(-1)
        probs = torch.softmax(logits.float() / t, -1).cpu()
        ids = ids.clone()
        for row in torch.nonzero(temperature.cpu() > 0).flatten().tolist():
            g = torch.Generator(device="cpu")
            g.manual_seed(int(seeds[row]) & 0x7FFFFFFFFFFFFFFF if seeds is not None else row)
            ids[row] = torch.multinomial(probs[row], 1, generator=g)[0]
    return ids + index_offset, vals


def attention(q, k_cache, v_cache, block_tables, q_lens, kv_lens, Hq, Hkv, D, scale, causal=True,
              return_lse=False):
    """Paged attention oracle. q: [T, Hq*D]; caches [nb, Hkv, bs, D];
    sequence i owns q rows [sum(q_lens[:i]), +q_lens[i]) whose positions are the last
    q_lens[i] positions of its kv_lens[i] keys."""
    T = q.shape[0]
    bs = k_cache.shape[2]
    out = torch.zeros(T, Hq * D, dtype=q.dtype, device=q.device)
    lse = torch.full((T, Hq), -math.inf, dtype=torch.float32, device=q.device)
    G = Hq // Hkv
    t0 = 0
    for i, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        if ql == 0:
            continue
        nblk = (kl + bs - 1) // bs
        blocks = block_tables[i, :nblk].long()
        k = k_cache[blocks].permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :kl].float()
        v = v_cache[blocks].permute(1, 0, 2, 3).reshape(Hkv, nblk * bs, D)[:, :kl].float()
        qi = q[t0:t0 + ql].view(ql, Hq, D).permute(1, 0, 2).float()  # [Hq, ql, D]
        k = k.repeat_interleave(G, 0)
        v = v.repeat_interleave(G, 0)
        s = torch.einsum("hqd,hkd->hqk", qi, k) * scale
        if causal:
            qpos = torch.arange(kl - ql, kl, device=q.device).view(1, ql, 1)
            kpos = torch.arange(kl, device=q.device).view(1, 1, kl)
            s = s.masked_fill(kpos > qpos, -math.inf)
        lse[t0:t0 + ql] = torch.logsumexp(s, -1).t()
        p = torch.softmax(s, -1)
        o = torch.einsum("hqk,hkd->hqd", p, v)
        out[t0:t0 + ql] = o.permute(1, 0, 2).reshape(ql, Hq * D).to(q.dtype)
        t0 += ql
    return (out, lse) if return_lse else out


def attention_contiguous(q, k, v, seq_lens, H, D, scale, causal=False):
    """Varlen attention over packed sequences (encoder). q/k/v: [T, H*D]."""
    T = q.shape[0]
    out = torch.zeros(T, H * D, dtype=q.dtype, device=q.device)
    t0 = 0
    for n in seq_lens:
        qi = q[t0:t0 + n].view(n, H, D).permute(1, 0, 2).float()
        ki = k[t0:t0 + n].view(n, H, D).permute(1, 0, 2).float()
        vi = v[t0:t0 + n].view(n, H, D).permute(1, 0, 2).float()
        s = torch.einsum("hqd,hkd->hqk", qi, ki) * scale
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1),
                              -math.inf)
        o = torch.einsum("hqk,hkd->hqd", torch.softmax(s, -1), vi)
        out[t0:t0 + n] = o.permute(1, 0, 2).reshape(n, H * D).to(q.dtype)
        t0 += n
    return out


def merge_attn_states(o1, lse1, o2, lse2):
    """Combine two attention results over disjoint key sets. o: [T, H, D], lse: [T, H]."""
    m = torch.maximum(lse1, lse2)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    den = (w1 + w2).clamp_min(1e-30)
    o = (o1.float() * w1.unsqueeze(-1) + o2.float() * w2.unsqueeze(-1)) / den.unsqueeze(-1)
    return o.to(o1.dtype), m + torch.log(den)
