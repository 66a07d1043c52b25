"""Rank topology and the collectives of the two execution modes.

Layout (reference: arctic_inference/vllm/ulysses.py:128-136,222-251): the ranks
of one engine form an SP x TP grid with TP fastest, ``rank = s * TP + t``.

* ``tp_group``   -- ranks that differ in ``t`` (row-parallel reductions in SP mode)
* ``sp_group``   -- ranks that differ in ``s`` (Ulysses exchanges)
* ``full_group`` -- all ``TP*SP`` ranks; rank (s, t) owns head block
  ``p = t * SP + s`` and, in shift (full tensor-parallel) mode, vocabulary shard p.

:class:`Communicator` is the library-collective implementation (NCCL on GPUs,
gloo on CPU): it is what the reference does and is kept as the A/B baseline and
as the CPU-testable statement of the data movement. :class:`FusedCommunicator`
(``fused.py``) overrides the hot exchanges with kernels that move the data over
NVLink from inside the compute kernels.

Sequence-parallel data flow of one attention layer
(arctic_inference/vllm/ulysses.py:418-457): each rank projects QKV for its
``n = N/SP`` tokens and all head blocks; the first exchange turns
``[n, SP*(h+2hkv)*D]`` into ``[N, (h+2hkv)*D]`` (all tokens, own heads, rows in
global token order because ranks hold contiguous token slices); attention runs
over all tokens with local heads; the second exchange turns ``[N, h*D]`` back
into ``[n, SP*h*D]``.
"""

from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..models.llama import ShardSpec


class Topology:
    def __init__(self, tp: int, sp: int, rank: int):
        self.tp, self.sp = tp, sp
        self.ways = tp * sp
        self.rank = rank
        self.tp_rank = rank % tp
        self.sp_rank = rank // tp
        self.head_block = self.tp_rank * sp + self.sp_rank

    def tp_group_ranks(self) -> list[int]:
        return [self.sp_rank * self.tp + t for t in range(self.tp)]

    def sp_group_ranks(self) -> list[int]:
        return [s * self.tp + self.tp_rank for s in range(self.sp)]

    @staticmethod
    def all_tp_groups(tp, sp):
        return [[s * tp + t for t in range(tp)] for s in range(sp)]

    @staticmethod
    def all_sp_groups(tp, sp):
        return [[s * tp + t for s in range(sp)] for t in range(tp)]

    def rank_of_block(self, p: int) -> int:
        t, s = divmod(p, self.sp)
        return s * self.tp + t

    def kv_replication(self, num_kv_heads: int) -> int:
        return max(1, self.ways // num_kv_heads)


class Communicator:
    """Library collectives (the baseline path)."""

    fused = False

    def __init__(self, tp: int, sp: int, device: Optional[torch.device] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.world = dist.get_world_size()
        if self.world != tp * sp:
            raise ValueError("world size %d != TP*SP = %d" % (self.world, tp * sp))
        self.topo = Topology(tp, sp, dist.get_rank())
        self.tp, self.sp, self.ways = tp, sp, tp * sp
        self.rank = self.topo.rank
        self.device = device
        self.full_group = dist.group.WORLD
        self.tp_group = self.sp_group = None
        # every rank must create every group, in the same order
        if tp > 1 and sp > 1:
            for ranks in Topology.all_tp_groups(tp, sp):
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.tp_group = g
            for ranks in Topology.all_sp_groups(tp, sp):
                g = dist.new_group(ranks)
                if self.rank in ranks:
                    self.sp_group = g
        elif tp > 1:
            self.tp_group = dist.group.WORLD
        elif sp > 1:
            self.sp_group = dist.group.WORLD
        self.stats = {"all_to_all": 0, "all_reduce": 0, "all_gather": 0}

    def shard_spec(self) -> ShardSpec:
        return ShardSpec(self.tp, self.sp, self.topo.tp_rank, self.topo.sp_rank)

    # ------------------------------------------------------------- token slicing
    def local_token_slice(self, t: torch.Tensor) -> torch.Tensor:
        n = t.shape[0] // self.sp
        s = self.topo.sp_rank
        return t[s * n:(s + 1) * n]

    # ----------------------------------------------------------- Ulysses exchange
    def qkv_scatter_heads(self, x_local, wqkv, blk_rows: int, bias=None) -> torch.Tensor:
        """[n, H] local tokens -> [N, blk_rows] all tokens x this rank's head block."""
        n = x_local.shape[0]
        qkv = ops.linear(x_local, wqkv, bias=bias)            # [n, SP*blk_rows]
        send = qkv.view(n, self.sp, blk_rows).transpose(0, 1).contiguous()  # [SP, n, blk]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv.view(self.sp * n, blk_rows), send.view(self.sp * n, blk_rows),
                               group=self.sp_group)
        self.stats["all_to_all"] += 1
        return recv.view(self.sp * n, blk_rows)

    def attention_gather_tokens(self, q, k_cache, v_cache, meta, h, hkv, D, scale):
        """Attention over all N tokens with local heads, then [N, h*D] -> [n, SP*h*D]."""
        attn = ops.attention(q, k_cache, v_cache, meta, h, hkv, D, scale)
        N = attn.shape[0]
        n = N // self.sp
        recv = torch.empty(self.sp, n, h * D, dtype=attn.dtype, device=attn.device)
        dist.all_to_all_single(recv.view(N, h * D), attn.contiguous(), group=self.sp_group)
        self.stats["all_to_all"] += 1
        return recv.transpose(0, 1).reshape(n, self.sp * h * D)

    def gather_rows_all(self, h_local, res_local, idx):
        """Rows ``idx`` (global token indices) of the token-sliced tensors, on every rank."""
        n = h_local.shape[0]
        s = self.topo.sp_rank
        B = idx.numel()
        H = h_local.shape[1]
        local = idx - s * n
        own = (local >= 0) & (local < n)
        buf = torch.zeros(2, B, H, dtype=torch.float32, device=h_local.device)
        sel = local.clamp(0, n - 1)
        buf[0] = h_local[sel].float() * own.unsqueeze(1)
        buf[1] = res_local[sel].float() * own.unsqueeze(1)
        dist.all_reduce(buf, group=self.sp_group)
        self.stats["all_reduce"] += 1
        return buf[0].to(h_local.dtype), buf[1].to(h_local.dtype).contiguous()

    def swiftkv_boundary(self, h_local, res_local, weight, eps: float, idx):
        """``res_local += h_local``; returns the SwiftKV-normalised hidden state of every token
        of the step ([N, H], on all ranks) and the updated residual rows of the sampled tokens
        ``idx`` (arctic_inference/vllm/swiftkv/llama_swiftkv.py:236-241 gathers both tensors
        whole; the later layers only read the residual at the sampled rows)."""
        s_local = ops.rmsnorm(h_local, weight, eps, residual=res_local)
        n, H = s_local.shape
        out = torch.empty(self.sp * n, H, dtype=s_local.dtype, device=s_local.device)
        dist.all_gather_into_tensor(out, s_local.contiguous(), group=self.sp_group)
        self.stats["all_gather"] += 1
        _, x_sel = self.gather_rows_all(res_local, res_local, idx)
        return out, x_sel

    # ---------------------------------------------------------------- reductions
    def all_reduce_full(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.full_group)
        self.stats["all_reduce"] += 1
        return t

    def all_reduce_tp(self, t: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(t, group=self.tp_group)
        self.stats["all_reduce"] += 1
        return t

    # ------------------------------------------------------------------ sampling
    def argmax_exchange(self, ids: torch.Tensor, vals: torch.Tensor) -> torch.Tensor:
        """Global arg-max from per-shard (best id, best value): 16 bytes per row per rank
        (reference: arctic_inference/vllm/fp32_lm_head.py:179-185)."""
        B = ids.numel()
        mine = torch.stack([vals.double(), ids.double()], 1).contiguous()   # [B, 2]
        allv = torch.empty(self.ways, B, 2, dtype=torch.float64, device=ids.device)
        dist.all_gather_into_tensor(allv.view(self.ways * B, 2), mine, group=self.full_group)
        self.stats["all_gather"] += 1
        v, i = allv[..., 0], allv[..., 1]
        best = v.max(0).values
        cand = torch.where(v == best.unsqueeze(0), i, torch.full_like(i, float("inf")))
        return cand.min(0).values.long()

    def gather_vocab(self, logits: torch.Tensor, vocab: int) -> torch.Tensor:
        """Full logits [B, V] from vocabulary shards (shard p lives on rank_of_block(p))."""
        B, per = logits.shape
        width = ((vocab + self.ways - 1) // self.ways + 7) // 8 * 8
        pad = torch.zeros(B, width, dtype=logits.dtype, device=logits.device)
        pad[:, :per] = logits
        allv = torch.empty(self.ways, B, width, dtype=logits.dtype, device=logits.device)
        dist.all_gather_into_tensor(allv.view(self.ways * B, width), pad, group=self.full_group)
        self.stats["all_gather"] += 1
        order = [self.topo.rank_of_block(p) for p in range(self.ways)]
        return allv[order].permute(1, 0, 2).reshape(B, self.ways * width)[:, :vocab]

    def barrier(self) -> None:
        dist.barrier()

    def broadcast_object(self, obj, src: int = 0):
        box = [obj]
        dist.broadcast_object_list(box, src=src)
        return box[0]

    def host_broadcast(self, obj, src: int = 0):
        """Broadcast a Python object over a host-side (gloo) group, off the GPU streams: the
        control channel of the serving loop. Every rank must call it in the same order."""
        if getattr(self, "_host_group", None) is None:
            if dist.get_backend() == "gloo":
                self._host_group = dist.group.WORLD
            else:
                self._host_group = dist.new_group(backend="gloo")
        box = [obj]
        dist.broadcast_object_list(box, src=src, group=self._host_group)
        return box[0]


def init_communicator(tp: int, sp: int, backend: str = "fused", device=None) -> Communicator:
    """Create the process group from torchrun-style environment variables (if needed)
    and return the communicator for this rank."""
    use_cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if use_cuda:
            local = int(os.environ.get("LOCAL_RANK", str(rank)))
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = None
    if use_cuda:
        dev = torch.device("cuda", torch.cuda.current_device())
    if backend == "fused" and use_cuda:
        from .fused import FusedCommunicator
        return FusedCommunicator(tp, sp, dev)
    return Communicator(tp, sp, dev)
