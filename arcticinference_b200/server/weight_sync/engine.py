"""Two-party tensor channel and the streaming protocol on top of it.

A channel is a private two-rank process group (NCCL when the tensors live on GPUs, gloo for
host tensors) that does not touch the process's default group: the sender listens on a TCP
port, the receiver connects, both construct the group from that store. One channel exists per
(replica, rank) pair, so replicas can be updated independently of each other
(reference: arctic_inference/server/weight_sync/engine.py:66-169, utils.py:32-79, where a
stateless group and pynccl play this role).

Stream layout (sender rank 0 -> receiver rank 1):

    header   int64[2]  = (MAGIC, number of plan bytes)
    plan     uint8[n]  = the TransferSchedule as UTF-8 JSON (TransferSchedule.to_json)
    direct tensors, one message each, in plan order
    buckets, one uint8 message each; the receiver keeps two bucket buffers so that bucket
             i+1 is in flight while the tensors of bucket i are being loaded
    ack      int64[1]  receiver -> sender: tensors applied

``reverse`` transfers run the same stream from rank 1 to rank 0.
"""

from __future__ import annotations

import logging
from datetime import timedelta
from typing import Callable, Iterator, Optional

import torch
import torch.distributed as dist

from .schedule import TransferSchedule, dtype_from_name

logger = logging.getLogger(__name__)

MAGIC = 0x41423230305753  # "AB200WS"
DEFAULT_TIMEOUT_S = 120.0
MAX_PLAN_BYTES = 64 << 20


class Alias(str):
    """Stands for a tensor that shares storage with the named one."""


class Channel:
    """rank 0 hosts the rendezvous store (the sender side by convention)."""

    def __init__(self, host: str, port: int, rank: int, device: Optional[torch.device] = None,
                 timeout: float = DEFAULT_TIMEOUT_S):
        self.rank, self.peer = rank, 1 - rank
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        td = timedelta(seconds=timeout)
        self.store = dist.TCPStore(host, port, 2, is_master=(rank == 0), timeout=td,
                                   wait_for_workers=False)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = td
            self.pg = dist.ProcessGroupNCCL(self.store, rank, 2, opts)
        else:
            self.pg = dist.ProcessGroupGloo(self.store, rank, 2, td)
        self._tag = 0

    def send(self, t: torch.Tensor):
        return self.pg.send([t], self.peer, 0)

    def recv(self, t: torch.Tensor):
        return self.pg.recv([t], self.peer, 0)

    def _ctl(self, n: int) -> torch.Tensor:
        return torch.zeros(n, dtype=torch.int64, device=self.device)

    def send_ints(self, *vals: int) -> None:
        t = self._ctl(len(vals))
        t.copy_(torch.tensor(vals, dtype=torch.int64))
        self.send(t).wait()

    def recv_ints(self, n: int) -> list:
        t = self._ctl(n)
        self.recv(t).wait()
        return [int(v) for v in t.cpu()]

    def send_bytes(self, b: bytes) -> None:
        t = torch.frombuffer(bytearray(b), dtype=torch.uint8).to(self.device)
        self.send(t).wait()

    def recv_bytes(self, n: int) -> bytes:
        t = torch.empty(n, dtype=torch.uint8, device=self.device)
        self.recv(t).wait()
        return bytes(t.cpu().numpy().tobytes())

    def close(self) -> None:
        self.pg = None
        self.store = None


def send_stream(ch: Channel, tensors: dict, schedule: TransferSchedule) -> int:
    """Send ``tensors`` (name -> tensor on ``ch.device`` or elsewhere) following ``schedule``.
    Returns the receiver's count of applied tensors."""
    plan = schedule.to_json().encode("utf-8")
    ch.send_ints(MAGIC, len(plan))
    ch.send_bytes(plan)
    for m in schedule.direct:
        t = tensors[m.name].to(ch.device).contiguous()
        ch.send(t).wait()
    bufs = [None, None]
    works = [None, None]
    size = schedule.max_bucket_bytes()
    if size:
        bufs = [torch.empty(size, dtype=torch.uint8, device=ch.device) for _ in range(2)]
    for i, b in enumerate(schedule.buckets):
        k = i & 1
        if works[k] is not None:
            works[k].wait()
        buf = bufs[k]
        for s in b.slots:
            src = tensors[s.meta.name].contiguous().view(-1).view(torch.uint8)
            buf[s.offset:s.offset + src.numel()].copy_(src, non_blocking=True)
        if ch.device.type == "cuda":
            torch.cuda.current_stream(ch.device).synchronize()
        works[k] = ch.send(buf[:b.nbytes])
    for w in works:
        if w is not None:
            w.wait()
    return ch.recv_ints(1)[0]


def receive_stream(ch: Channel, direct_target: Optional[Callable] = None) -> Iterator:
    """Yield (name, tensor) for every tensor of the stream. Bucketed tensors are views of a
    bucket buffer that is reused two buckets later: consume (copy) each before asking for the
    next. ``direct_target(meta)`` may return the destination tensor of a direct transfer (it is
    then received in place and yielded as is); otherwise a fresh tensor is allocated.
    Send the closing ack with :func:`ack`."""
    magic, n = ch.recv_ints(2)
    if magic != MAGIC:
        raise RuntimeError("weight stream: bad magic %x" % magic)
    if n < 0 or n > MAX_PLAN_BYTES:
        raise RuntimeError("weight stream: plan of %d bytes refused" % n)
    schedule = TransferSchedule.from_json(ch.recv_bytes(n).decode("utf-8"))
    for m in schedule.direct:
        dst = direct_target(m) if direct_target is not None else None
        ok = dst is not None and tuple(dst.shape) == tuple(m.shape) and \
            dst.dtype == dtype_from_name(m.dtype) and dst.is_contiguous() and dst.device == ch.device
        if not ok:
            dst = torch.empty(m.shape, dtype=dtype_from_name(m.dtype), device=ch.device)
        ch.recv(dst).wait()
        yield m.name, dst
    size = schedule.max_bucket_bytes()
    if schedule.buckets:
        bufs = [torch.empty(size, dtype=torch.uint8, device=ch.device) for _ in range(2)]
        work = ch.recv(bufs[0][:schedule.buckets[0].nbytes])
        for i, b in enumerate(schedule.buckets):
            work.wait()
            if i + 1 < len(schedule.buckets):
                work = ch.recv(bufs[(i + 1) & 1][:schedule.buckets[i + 1].nbytes])
            buf = bufs[i & 1]
            for s in b.slots:
                m = s.meta
                dt = dtype_from_name(m.dtype)
                yield m.name, buf[s.offset:s.offset + m.nbytes].view(dt).view(m.shape)
    for m in schedule.aliases:
        yield m.name, Alias(m.alias_of)     # tied: the consumer re-links it to that tensor


def ack(ch: Channel, applied: int) -> None:
    ch.send_ints(applied)
