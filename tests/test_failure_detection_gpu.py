"""Device-side waits are bounded: a peer that never arrives turns into an error status that
the host reads, and the context stays usable. The "missing peer" is a flag slot in this GPU's
own memory that nothing writes, so no second GPU (and no fault) is involved."""

import time

import pytest
import torch

from arcticinference_b200 import ops
from arcticinference_b200.ops.native import KernelTimeout

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_barrier_times_out_when_a_peer_never_arrives():
    mine = torch.zeros(16, dtype=torch.int32, device=DEV)       # rank 0's arrival slots
    peer = torch.zeros(16, dtype=torch.int32, device=DEV)       # stands in for rank 1's
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.check_status()
    t0 = time.time()
    ops.peer_barrier([mine, peer], 0, epoch, limit_ms=200)
    with pytest.raises(KernelTimeout, match="peer flag"):
        ops.check_status()
    assert 0.15 < time.time() - t0 < 5.0
    assert int(peer[0]) == 1 and int(mine[0]) == 1              # our own arrival was published
    # the host plays the missing rank: once its flag is there the same barrier completes
    mine[1] = 2
    ops.peer_barrier([mine, peer], 0, epoch, limit_ms=200)
    ops.check_status()
    assert int(epoch) == 2
    # and the GPU keeps working
    x = (torch.randn(64, 256, device=DEV)).to(torch.bfloat16)
    w = (torch.randn(128, 256, device=DEV) * 0.05).to(torch.bfloat16)
    y = ops.linear(x, w)
    ops.check_status()
    assert torch.isfinite(y.float()).all()


def test_single_rank_barrier_is_immediate():
    mine = torch.zeros(16, dtype=torch.int32, device=DEV)
    epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
    for i in range(3):
        ops.peer_barrier([mine], 0, epoch, limit_ms=100)
    ops.check_status()
    assert int(epoch) == 3 and int(mine[0]) == 3
