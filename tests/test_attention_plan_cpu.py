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


def test_tail_split_plan_cuts_the_last_round_only():
    # 128 sequences x 8 KV heads on 296 CTA slots: three full waves and 136 CTAs in a fourth;
    # the 17 sequences of that wave are cut in two so that their pieces cover the slots
    assert ops.tail_split_plan(128, 8, 296) == (17, 2)
    assert ops.tail_split_plan(64, 8, 296) == (0, 1)     # last wave 73 % full: left alone
    assert ops.tail_split_plan(37, 8, 296) == (0, 1)     # exactly one wave
    assert ops.tail_split_plan(16, 8, 296) == (0, 1)     # fewer CTAs than slots: other rule


def test_large_decode_batch_cuts_its_longest_sequences_and_places_the_pieces_last():
    kv = [2000 + i for i in range(128)]
    work, tok_splits, max_splits = ops.plan_attention_work([1] * 128, kv, 4, True, Hkv=8)
    assert max_splits == 2 and work.shape == (128 + 17, 8)
    assert sorted(np.nonzero(tok_splits == 2)[0].tolist()) == list(range(111, 128))
    _covered(work, 128, kv)
    lengths = work[:, 5] - work[:, 4]
    assert all(a >= b for a, b in zip(lengths, lengths[1:]))       # heaviest first
    assert set(work[-34:, 0].tolist()) == set(range(111, 128))      # the pieces come last
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
