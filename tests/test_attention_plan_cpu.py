"""The host-side planner of attention work items (``ops.plan_attention_work``)."""

import numpy as np

from arcticinference_b200 import ops


def _covered(work, n_seq, kv_lens):
    """Every sequence's keys are covered exactly once by its work items."""
    got = {i: [] for i in range(n_seq)}
    for seq, tok, n, qpos, ks, ke, si, ns in work:
        if n > 0:
            got[int(seq)].append((int(ks), int(ke), int(si), int(ns)))
    for i, kl in enumerate(kv_lens):
        spans = sorted(got[i])
        assert spans[0][0] == 0 and spans[-1][1] >= kl
        for (a0, a1, _, _), (b0, _b1, _, _) in zip(spans, spans[1:]):
            assert a1 == b0
        assert all(ns == len(spans) for _, _, _, ns in spans)
        assert sorted(si for _, _, si, _ in spans) == list(range(len(spans)))


def test_large_decode_batch_keeps_sequences_whole():
    # more CTAs than the GPU holds at once: no split (measured: halving the sequences of a
    # 128 x 2000 batch to even out the rounds of CTAs did not shorten the call)
    kv = [2000] * 128
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 128, kv, 4, True, Hkv=8)
    assert max_splits == 1 and work.shape == (128, 8)
    _covered(work, 128, kv)


def test_small_decode_batch_is_split_to_occupy_the_gpu():
    kv = [4000] * 16
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 16, kv, 4, True, Hkv=8)
    assert max_splits > 1
    _covered(work, 16, kv)
    assert np.all(work[:, 2] == 1)
