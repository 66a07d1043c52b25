"""Sending side of a weight update: runs in the trainer (or any process that holds the new
parameters under checkpoint names).

    sender = WeightSender(named_tensors)                     # dict name -> tensor
    sender.send(groups=[{"master_addr": "10.0.0.5", "master_port": 41000,
                         "replica_ids": [0, 1]}], ranks_per_replica=1)

For every (replica, rank) the sender opens the listening side of a private channel on
``master_port + replica_id * ranks_per_replica + rank`` and streams all tensors; replicas are
served concurrently, one thread per channel. The replicas are told to connect through the
pool's ``sync_weights`` (REST: ``POST /sync_weights`` with the same groups).
(reference: arctic_inference/server/weight_sync/sender.py:131-203.)
"""

from __future__ import annotations

import threading
import time
from typing import Iterable, Optional

import torch

from .engine import Channel, ack, receive_stream, send_stream
from .schedule import TensorMeta, TransferSchedule, find_aliases


class WeightSender:
    def __init__(self, named_tensors, device: Optional[str] = None, direct_names: Iterable[str] = ()):
        self.tensors = dict(named_tensors)
        self.device = torch.device(device) if device is not None else \
            next(iter(self.tensors.values())).device
        self.direct_names = set(direct_names)
        self.last_stats: list = []

    def build_schedule(self, bucket_size: int = 256 << 20) -> TransferSchedule:
        al = find_aliases(self.tensors)
        metas = []
        for n, t in self.tensors.items():
            m = TensorMeta.of(n, t, direct=n in self.direct_names)
            m.alias_of = al.get(n)
            metas.append(m)
        return TransferSchedule.build(metas, bucket_size)

    def _serve(self, host: str, port: int, sched: TransferSchedule, timeout: float, out: list,
               reverse: bool) -> None:
        t0 = time.time()
        try:
            ch = Channel(host, port, rank=0, device=self.device, timeout=timeout)
            try:
                if reverse:
                    got = {}
                    for name, t in receive_stream(ch):
                        got[name] = t if isinstance(t, str) else t.clone()
                    ack(ch, len(got))
                    out.append({"port": port, "received": got, "seconds": time.time() - t0})
                else:
                    applied = send_stream(ch, self.tensors, sched)
                    out.append({"port": port, "applied": applied, "bytes": sched.total_bytes,
                                "seconds": time.time() - t0})
            finally:
                ch.close()
        except BaseException as e:  # noqa: BLE001 - reported to the caller of send()
            out.append({"port": port, "error": "%s: %s" % (type(e).__name__, e)})

    def start(self, groups: list, ranks_per_replica: int = 1, bucket_size: int = 256 << 20,
              timeout: float = 120.0, bind_host: Optional[str] = None, reverse: bool = False) -> list:
        """Open every channel in a background thread; returns the threads. Call ``join``."""
        sched = self.build_schedule(bucket_size)
        self.last_stats = []
        threads = []
        for g in groups:
            host = bind_host or g["master_addr"]
            for rid in g["replica_ids"]:
                for r in range(ranks_per_replica):
                    port = int(g["master_port"]) + rid * ranks_per_replica + r
                    th = threading.Thread(target=self._serve, daemon=True,
                                          args=(host, port, sched, timeout, self.last_stats, reverse))
                    th.start()
                    threads.append(th)
        return threads

    def start_ports(self, host: str, ports: Iterable[int], bucket_size: int = 256 << 20,
                    timeout: float = 120.0, reverse: bool = False) -> list:
        """One channel per port (a trainer rank's share of a :class:`SenderSchedule`:
        ``plan.ports_of(train_rank, base_port)``); returns the threads. Call ``join``."""
        sched = self.build_schedule(bucket_size)
        self.last_stats = []
        threads = []
        for port in ports:
            th = threading.Thread(target=self._serve, daemon=True,
                                  args=(host, int(port), sched, timeout, self.last_stats, reverse))
            th.start()
            threads.append(th)
        return threads

    def join(self, threads: list) -> list:
        for th in threads:
            th.join()
        bad = [s for s in self.last_stats if "error" in s]
        if bad:
            raise RuntimeError("weight transfer failed on port %d: %s" % (bad[0]["port"], bad[0]["error"]))
        return self.last_stats

    def send(self, groups: list, **kw) -> list:
        return self.join(self.start(groups, **kw))
