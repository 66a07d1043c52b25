"""Forest-cascade planning: grouping, gates, and equivalence of the cascaded work list with
plain attention (the work list is interpreted by a small PyTorch restatement of the kernel)."""

import math

import numpy as np
import pytest
import torch

from arcticinference_b200.config import ForestCascadeConfig
from arcticinference_b200.engine import forest_cascade as fca
from arcticinference_b200.ops import reference as ref

BS = 16


def _run_work(q, kc, vc, table, work, tok_splits, Hq, Hkv, D, scale):
    """Execute attention work items like csrc/attention.cu does, merging partials by LSE."""
    T = q.shape[0]
    G = Hq // Hkv
    parts = {}
    for seq, t0, n, qpos0, ks, ke, split, ns in work.tolist():
        if n <= 0:
            continue
        ke = min(ke, qpos0 + n)
        nblk = (ke + BS - 1) // BS
        blocks = torch.as_tensor(table[seq, :nblk]).long()
        k = kc[blocks].permute(1, 0, 2, 3).reshape(Hkv, nblk * BS, D)[:, ks:ke].float()
        v = vc[blocks].permute(1, 0, 2, 3).reshape(Hkv, nblk * BS, D)[:, ks:ke].float()
        qi = q[t0:t0 + n].view(n, Hq, D).permute(1, 0, 2).float()
        s = torch.einsum("hqd,hkd->hqk", qi, k.repeat_interleave(G, 0)) * scale
        qpos = (qpos0 + torch.arange(n)).view(1, n, 1)
        kpos = (ks + torch.arange(ke - ks)).view(1, 1, -1)
        s = s.masked_fill(kpos > qpos, -math.inf)
        lse = torch.logsumexp(s, -1)
        o = torch.einsum("hqk,hkd->hqd", torch.softmax(s, -1), v.repeat_interleave(G, 0))
        for j in range(n):
            parts.setdefault(t0 + j, []).append((o[:, j], lse[:, j]))
    out = torch.zeros(T, Hq, D)
    for t, ps in parts.items():
        m = torch.stack([l for _, l in ps]).max(0).values
        w = [torch.exp(l - m) for _, l in ps]
        out[t] = sum(wi.unsqueeze(-1) * o for wi, (o, _) in zip(w, ps)) / sum(w).unsqueeze(-1)
        assert len(ps) == tok_splits[t]
    return out.reshape(T, Hq * D)


def _batch(rng, shared):
    """Requests built from shared prefixes: `shared` = list of (num_requests, prefix_blocks)."""
    tables, ctx = [], []
    next_block = 1
    for n, pre in shared:
        prefix = list(range(next_block, next_block + pre))
        next_block += pre
        for _ in range(n):
            own = int(rng.integers(1, 4))
            t = prefix + list(range(next_block, next_block + own))
            next_block += own
            tables.append(t)
            ctx.append(len(t) * BS - int(rng.integers(1, BS)))  # last block partly filled
    return tables, ctx, next_block


def test_grouping_finds_shared_prefixes():
    rng = np.random.default_rng(0)
    tables, ctx, _ = _batch(rng, [(6, 10), (4, 3), (1, 0), (5, 7)])
    perm = rng.permutation(len(tables))
    tables = [tables[i] for i in perm]
    ctx = [ctx[i] for i in perm]
    plan = fca.plan_groups(tables, ctx, BS, ForestCascadeConfig(enabled=True, min_batch_size=4))
    assert plan is not None
    found = sorted((len(g.members), g.prefix_blocks) for g in plan.non_singleton)
    assert found == [(4, 3), (5, 7), (6, 10)]
    assert plan.saved_block_reads == 5 * 10 + 3 * 3 + 4 * 7
    assert sorted(plan.order) == list(range(len(tables)))


def test_gates():
    rng = np.random.default_rng(1)
    cfg = ForestCascadeConfig(enabled=True, min_batch_size=8)
    tables, ctx, _ = _batch(rng, [(3, 5)])
    assert fca.plan_groups(tables, ctx, BS, cfg) is None                    # batch too small
    tables, ctx, _ = _batch(rng, [(1, 0)] * 10)
    assert fca.plan_groups(tables, ctx, BS, cfg) is None                    # nothing shared
    tables, ctx, _ = _batch(rng, [(2, 4)] + [(1, 0)] * 14)
    assert fca.plan_groups(tables, ctx, BS, cfg) is None                    # too few grouped
    assert not fca.gate(cfg, [1] * 4, True) and fca.gate(cfg, [1] * 9, True)
    assert not fca.gate(cfg, [40] * 9, True) and not fca.gate(cfg, [1] * 9, False)
    assert ForestCascadeConfig.from_json(None).enabled is False
    assert ForestCascadeConfig.from_json("{}").enabled is True
    assert ForestCascadeConfig.from_json('{"min_group_size": 3}').min_group_size == 3
    with pytest.raises(ValueError):
        ForestCascadeConfig.from_json('{"bogus": 1}')


@pytest.mark.parametrize("q_len", [1, 3])
def test_cascade_work_equals_plain_attention(q_len):
    rng = np.random.default_rng(2)
    torch.manual_seed(0)
    Hq, Hkv, D = 4, 2, 32
    tables, ctx, nb = _batch(rng, [(5, 6), (3, 2), (2, 0)])
    cfg = ForestCascadeConfig(enabled=True, min_batch_size=4)
    plan = fca.plan_groups(tables, ctx, BS, cfg)
    assert plan is not None
    tables = [tables[i] for i in plan.order]
    kv_lens = [ctx[i] + q_len for i in plan.order]
    # the last block must have room for the query tokens
    kv_lens = [min(k, len(t) * BS) for k, t in zip(kv_lens, tables)]
    q_lens = [q_len] * len(tables)
    work, tok_splits, table, max_splits = fca.build_cascade_work(plan, q_lens, kv_lens, tables, BS,
                                                                 Hq // Hkv)
    assert max_splits == 2 and int(tok_splits.max()) == 2
    T = sum(q_lens)
    q = torch.randn(T, Hq * D)
    kc, vc = torch.randn(nb, Hkv, BS, D), torch.randn(nb, Hkv, BS, D)
    got = _run_work(q, kc, vc, table, work, tok_splits, Hq, Hkv, D, 1 / math.sqrt(D))
    width = max(len(t) for t in tables)
    full = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        full[i, :len(t)] = torch.tensor(t)
    exp = ref.attention(q, kc, vc, full, q_lens, kv_lens, Hq, Hkv, D, 1 / math.sqrt(D)).float()
    assert torch.allclose(got, exp, atol=1e-4, rtol=1e-4)
