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


def test_wave_splits_fills_the_last_round():
    # 1024 CTAs on 296 slots: four rounds for the work of 3.46; two pieces per sequence make
    # seven rounds for 6.92
    assert ops.wave_splits(1024, 296) == 2
    assert ops.wave_splits(2048, 296) == 1      # already 6.92 of 7
    assert ops.wave_splits(296, 296) == 1
    assert ops.wave_splits(512, 296) == 4
    assert ops.wave_splits(512, 296, max_splits=2) == 1


def test_large_decode_batch_is_split_to_even_out_rounds():
    kv = [2000] * 128
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 128, kv, 4, True, Hkv=8)
    assert max_splits == 2 and work.shape == (256, 8)
    assert (tok_splits == 2).all()
    _covered(work, 128, kv)
    # short sequences stay whole
    kv2 = [2000] * 64 + [300] * 64
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 128, kv2, 4, True, Hkv=8)
    assert list(tok_splits[:64]) == [2] * 64 and list(tok_splits[64:]) == [1] * 64
    _covered(work, 128, kv2)
    # a cap of one split (a captured graph without partial buffers) is respected
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 128, kv, 4, True, Hkv=8,
                                                           max_splits_cap=1)
    assert max_splits == 1 and work.shape[0] == 128


def test_small_decode_batch_is_split_to_occupy_the_gpu():
    kv = [4000] * 16
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 16, kv, 4, True, Hkv=8)
    assert max_splits > 1
    _covered(work, 16, kv)
    assert np.all(work[:, 2] == 1)
