"""Pipeline parallelism over whole-model stages (``--pipeline-parallel-size P`` with TP = SP = 1).

Stage ``s`` of ``P`` owns the decoder layers ``pipeline_layer_range(L, s, P)``, their KV cache,
the embedding table when it is the first stage, and the final norm and LM head when it is the
last. Every rank runs the same scheduler on the same request stream (as with the other
parallel modes), so batch composition, block tables and slot mappings agree without being
sent; what travels per step is the hidden state and the residual stream from one stage to the
next (point-to-point) and the sampled token ids from the last stage to all (a broadcast).

A step is one batch walking through the stages, so the stages of one replica work one after
the other: this form scales memory (a model that does not fit one GPU), not throughput; the
reference gets its pipeline schedule from vLLM's executor
(arctic_inference/vllm/ulysses.py:72-90,177-220 only lays out the groups).
Transfers use ``torch.distributed`` point-to-point calls (NCCL on GPUs, gloo on CPU ranks).
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .layout import pipeline_layer_range


class PipelineComm:
    """Stage bookkeeping and the three transfers of a pipeline-parallel step."""

    def __init__(self, stages: int, device: Optional[torch.device] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        if dist.get_world_size() != stages:
            raise ValueError("pipeline_parallel_size (%d) must equal the number of ranks (%d)"
                             % (stages, dist.get_world_size()))
        self.stages = stages
        self.stage = dist.get_rank()
        self.rank = self.stage
        self.world = stages
        self.device = device
        # within a stage nothing is sharded: the model code sees a one-rank layout
        self.tp = self.sp = self.ways = 1
        self.fused = False
        self.stats = {"send": 0, "recv": 0, "broadcast": 0}
        self._host_group = None

    def shard_spec(self):
        from ..models.llama import ShardSpec
        return ShardSpec()

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.stages - 1

    def layer_range(self, num_layers: int) -> tuple[int, int]:
        return pipeline_layer_range(num_layers, self.stage, self.stages)

    # ------------------------------------------------------------------ transfers
    def send_hidden(self, h: torch.Tensor, residual: torch.Tensor) -> None:
        """Hand the layer output and the residual stream to the next stage (one message)."""
        both = torch.stack((h, residual)).contiguous()
        dist.send(both, dst=self.stage + 1)
        self.stats["send"] += 1

    def recv_hidden(self, num_tokens: int, hidden: int, dtype: torch.dtype, device):
        both = torch.empty(2, num_tokens, hidden, dtype=dtype, device=device)
        dist.recv(both, src=self.stage - 1)
        self.stats["recv"] += 1
        return both[0], both[1]

    def broadcast_ids(self, ids: Optional[torch.Tensor], count: int, device) -> torch.Tensor:
        """The sampled token ids of the step, from the last stage to every stage."""
        if ids is None:
            ids = torch.empty(count, dtype=torch.int64, device=device)
        dist.broadcast(ids, src=self.stages - 1)
        self.stats["broadcast"] += 1
        return ids

    def host_broadcast(self, obj, src: int = 0):
        """Python object from ``src`` to every stage over a host-side (gloo) group: the control
        channel of the serving loop."""
        if self._host_group is None:
            self._host_group = (dist.group.WORLD if dist.get_backend() == "gloo"
                                else dist.new_group(backend="gloo"))
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self._host_group)
        return box[0]

    broadcast_object = host_broadcast

    def min_over_stages(self, value: int, device) -> int:
        """The smallest of the stages' values (they must agree on the number of KV blocks)."""
        t = torch.tensor([value], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t.item())

    def barrier(self) -> None:
        dist.barrier()


def init_pipeline(stages: int, device: Optional[str] = None) -> PipelineComm:
    """Join the job's process group (one rank per stage; RANK / WORLD_SIZE / MASTER_* from the
    environment) and return this rank's :class:`PipelineComm`."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    use_cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
    dev = None
    if use_cuda:
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    return PipelineComm(stages, dev)
