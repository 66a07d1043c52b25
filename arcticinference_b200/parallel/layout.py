"""Rank layout of a whole deployment and the process groups cut out of it.

The ranks of a job form a six-dimensional grid, slowest to fastest dimension:

    external DP x DP x PP x PCP x SP x TP

(reference: arctic_inference/vllm/ulysses.py:128-136). A group "along" a dimension
is the set of ranks that agree in every other coordinate. Two groups are not of
that plain kind:

* ``sp_tp`` -- the SP x TP plane of one engine enumerated TP-major, i.e. position
  ``t * SP + s`` in the group is rank ``(s, t)``. Full tensor parallelism over
  this ordering gives rank (s, t) the same head block in shift mode as Ulysses
  attention gives it in sequence-parallel mode, which is why both modes can share
  one KV cache (ulysses.py:237-251).
* ``ep``    -- expert parallelism spans DP x PCP x TP for a fixed SP index and
  pipeline stage (ulysses.py:207-220).
* ``dcp``   -- decode context parallelism subdivides each TP group into runs of
  ``dcp`` consecutive ranks (ulysses.py:150-160).

The class only enumerates ranks (numpy, no process group is created), so that it
can be checked on a machine without GPUs; :func:`create_groups` turns the lists
into ``torch.distributed`` groups. The engine in this package executes the
SP x TP plane (``parallel/comm.py``, ``parallel/fused.py``); data-parallel
replicas are separate engines behind the replica pool.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

_DIMS = ("external_dp", "dp", "pp", "pcp", "sp", "tp")


@dataclass(frozen=True)
class RankCoords:
    external_dp: int
    dp: int
    pp: int
    pcp: int
    sp: int
    tp: int


class RankLayout:
    def __init__(self, tp: int = 1, sp: int = 1, pp: int = 1, dp: int = 1, pcp: int = 1,
                 external_dp: int = 1, dcp: int = 1, world_size: Optional[int] = None):
        sizes = dict(external_dp=external_dp, dp=dp, pp=pp, pcp=pcp, sp=sp, tp=tp)
        for k, v in sizes.items():
            if v < 1:
                raise ValueError("%s must be >= 1" % k)
        if dcp < 1 or tp % dcp:
            raise ValueError("dcp must divide tp")
        n = int(np.prod(list(sizes.values())))
        if world_size is not None and world_size != n:
            raise ValueError("world size %d != product of the parallel sizes %d" % (world_size, n))
        self.sizes = sizes
        self.dcp = dcp
        self.world_size = n
        self.grid = np.arange(n, dtype=np.int64).reshape([sizes[d] for d in _DIMS])

    # ----------------------------------------------------------------- coordinates
    def coords(self, rank: int) -> RankCoords:
        idx = np.unravel_index(rank, self.grid.shape)
        return RankCoords(*[int(i) for i in idx])

    def rank_of(self, **coords) -> int:
        idx = tuple(int(coords.get(d, 0)) for d in _DIMS)
        return int(self.grid[idx])

    def head_block(self, rank: int) -> int:
        """Index of the attention-head block (and shift-mode vocabulary shard) of a rank."""
        c = self.coords(rank)
        return c.tp * self.sizes["sp"] + c.sp

    def pp_stage(self, rank: int) -> int:
        return self.coords(rank).pp

    # ---------------------------------------------------------------------- groups
    def _along(self, dim: str) -> list[list[int]]:
        ax = _DIMS.index(dim)
        g = np.moveaxis(self.grid, ax, -1).reshape(-1, self.sizes[dim])
        return g.tolist()

    def tp_groups(self): return self._along("tp")
    def sp_groups(self): return self._along("sp")
    def pp_groups(self): return self._along("pp")
    def dp_groups(self): return self._along("dp")
    def pcp_groups(self): return self._along("pcp")

    def dcp_groups(self) -> list[list[int]]:
        return self.grid.reshape(-1, self.dcp).tolist()

    def sp_tp_groups(self) -> list[list[int]]:
        # swap the two fastest axes, then flatten the plane: TP-major order
        plane = self.sizes["sp"] * self.sizes["tp"]
        return np.swapaxes(self.grid, 4, 5).reshape(-1, plane).tolist()

    def ep_groups(self) -> list[list[int]]:
        # fixed (external DP, SP, PP); members enumerate DP, PCP, TP
        s = self.sizes
        g = np.transpose(self.grid, (0, 4, 2, 1, 3, 5))
        return g.reshape(-1, s["dp"] * s["pcp"] * s["tp"]).tolist()

    def all_groups(self) -> dict[str, list[list[int]]]:
        return {"tp": self.tp_groups(), "dcp": self.dcp_groups(), "pcp": self.pcp_groups(),
                "pp": self.pp_groups(), "dp": self.dp_groups(), "ep": self.ep_groups(),
                "sp": self.sp_groups(), "sp_tp": self.sp_tp_groups()}

    def groups_of(self, rank: int) -> dict[str, list[int]]:
        """The one group of every kind that contains ``rank``."""
        out = {}
        for name, groups in self.all_groups().items():
            for g in groups:
                if rank in g:
                    out[name] = g
                    break
        return out

    def kv_replication(self, num_kv_heads: int) -> int:
        """How many ranks of the SP x TP plane hold a copy of the same KV head
        (ulysses.py:290-294, 409-412)."""
        return max(1, self.sizes["sp"] * self.sizes["tp"] // num_kv_heads)

    def kv_head_of(self, rank: int, num_kv_heads: int) -> int:
        """First global KV head that ``rank`` holds; the same in both execution modes."""
        ways = self.sizes["sp"] * self.sizes["tp"]
        p = self.head_block(rank)
        if num_kv_heads >= ways:
            return p * (num_kv_heads // ways)
        return p // (ways // num_kv_heads)


def pipeline_layer_range(num_layers: int, pp_rank: int, pp_size: int) -> tuple[int, int]:
    """Layers ``[start, end)`` of one pipeline stage. Layers divide evenly; when they do not,
    the surplus goes one layer each to the stages just before the last one, which also
    carries the final norm and the LM head (the first stage carries the embedding)."""
    if not 0 <= pp_rank < pp_size:
        raise ValueError("pp_rank out of range")
    base, extra = divmod(num_layers, pp_size)
    counts = [base] * pp_size
    # stages pp_size-2, pp_size-3, ... take the surplus; with one stage there is none
    j = pp_size - 2
    while extra > 0:
        counts[j if j >= 0 else pp_size - 1] += 1
        j = j - 1 if j > 0 else pp_size - 2
        extra -= 1
    start = sum(counts[:pp_rank])
    return start, start + counts[pp_rank]


def pipeline_stage_of_rank(rank: int, tp: int, sp: int, pp: int) -> int:
    """Stage of a global rank: the SP x TP plane is the fastest-varying block of the layout
    (ulysses.py:72-90)."""
    return (rank // (tp * sp)) % pp


def create_groups(layout: RankLayout, rank: int, backend: Optional[str] = None) -> dict:
    """Create every process group of the layout (all ranks must call this, in the same
    order) and return the ones ``rank`` belongs to, keyed like :meth:`all_groups`."""
    import torch.distributed as dist
    mine = {}
    for name, groups in layout.all_groups().items():
        for ranks in groups:
            g = dist.new_group(ranks, backend=backend) if len(ranks) > 1 else None
            if rank in ranks:
                mine[name] = (g, ranks)
    return mine
