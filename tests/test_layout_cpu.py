"""Rank layout: group enumeration, head-block ownership, pipeline layer ranges."""

import itertools

import pytest

from arcticinference_b200.parallel.comm import Topology
from arcticinference_b200.parallel.layout import (RankLayout, pipeline_layer_range,
                                                  pipeline_stage_of_rank)


def test_plain_groups_partition_the_world():
    lay = RankLayout(tp=2, sp=2, pp=2, dp=2)
    assert lay.world_size == 16
    for name, groups in lay.all_groups().items():
        flat = sorted(r for g in groups for r in g)
        assert flat == list(range(16)), name
    # TP is the fastest dimension, SP the next one
    assert lay.tp_groups()[0] == [0, 1]
    assert lay.sp_groups()[0] == [0, 2]
    assert lay.pp_groups()[0] == [0, 4]
    assert lay.dp_groups()[0] == [0, 8]


def test_shift_group_is_tp_major_and_keeps_head_blocks():
    tp, sp = 2, 4
    lay = RankLayout(tp=tp, sp=sp)
    (group,) = lay.sp_tp_groups()
    assert group == [0, 2, 4, 6, 1, 3, 5, 7]
    for pos, rank in enumerate(group):
        # position in the shift group == head block in sequence-parallel mode
        assert lay.head_block(rank) == pos
        topo = Topology(tp, sp, rank)
        assert topo.head_block == pos and topo.rank_of_block(pos) == rank


def test_kv_head_ownership_agrees_between_modes():
    lay = RankLayout(tp=2, sp=8)           # 16 ranks, 8 kv heads -> replication 2
    assert lay.kv_replication(8) == 2
    heads = [lay.kv_head_of(r, 8) for r in lay.sp_tp_groups()[0]]
    assert heads == [0, 0, 1, 1, 2, 2, 3, 3, 4, 4, 5, 5, 6, 6, 7, 7]
    lay = RankLayout(tp=1, sp=4)
    assert [lay.kv_head_of(r, 8) for r in range(4)] == [0, 2, 4, 6]


def test_expert_and_context_groups():
    lay = RankLayout(tp=4, sp=2, dp=2, dcp=2)
    ep = lay.ep_groups()
    assert len(ep) == 2 and all(len(g) == 8 for g in ep)
    for g in ep:                            # one SP index per expert-parallel group
        assert len({lay.coords(r).sp for r in g}) == 1
        assert {lay.coords(r).dp for r in g} == {0, 1}
    for g in lay.dcp_groups():
        assert len(g) == 2 and g[1] == g[0] + 1
        assert lay.coords(g[0]).sp == lay.coords(g[1]).sp
    with pytest.raises(ValueError):
        RankLayout(tp=4, dcp=3)
    with pytest.raises(ValueError):
        RankLayout(tp=2, sp=2, world_size=8)


def test_groups_of_and_coords_roundtrip():
    lay = RankLayout(tp=2, sp=2, pp=3, pcp=2)
    for r in range(lay.world_size):
        c = lay.coords(r)
        assert lay.rank_of(external_dp=c.external_dp, dp=c.dp, pp=c.pp, pcp=c.pcp, sp=c.sp,
                           tp=c.tp) == r
        mine = lay.groups_of(r)
        assert set(mine) == {"tp", "dcp", "pcp", "pp", "dp", "ep", "sp", "sp_tp"}
        assert all(r in g for g in mine.values())
        assert pipeline_stage_of_rank(r, 2, 2, 3) == (r // 4) % 3


@pytest.mark.parametrize("layers,pp", list(itertools.product([32, 33, 34, 80, 7], [1, 2, 3, 4])))
def test_pipeline_layer_ranges_cover_all_layers(layers, pp):
    spans = [pipeline_layer_range(layers, r, pp) for r in range(pp)]
    assert spans[0][0] == 0 and spans[-1][1] == layers
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 == b0
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1
    if pp > 1 and layers % pp:
        assert sizes[-1] == min(sizes)      # the stage with the LM head takes no surplus


def _group_worker(rank, world, port, q):
    import os
    import torch
    import torch.distributed as dist
    from arcticinference_b200.parallel.layout import RankLayout, create_groups
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lay = RankLayout(tp=2, sp=2, world_size=world)
    groups = create_groups(lay, rank, backend="gloo")
    got = {}
    for name in ("tp", "sp", "sp_tp"):
        g, ranks = groups[name]
        t = torch.tensor([1 << rank])
        dist.all_reduce(t, group=g)
        got[name] = (int(t), ranks)
    q.put((rank, got))
    dist.barrier()
    dist.destroy_process_group()


def test_process_groups_are_created_as_enumerated():
    import torch.multiprocessing as mp
    from _mp_util import free_port
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_group_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(4))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, got in res.items():
        for name, (mask, ranks) in got.items():
            assert rank in ranks and mask == sum(1 << r for r in ranks), (rank, name, mask, ranks)
    assert res[0]["tp"][1] == [0, 1] and res[0]["sp"][1] == [0, 2]
    assert res[3]["sp_tp"][1] == [0, 2, 1, 3]
