"""Transfer plans: which trainer rank feeds which serving rank (:class:`SenderSchedule`), and
which tensor travels in which bucket at which offset (:class:`TransferSchedule`).

Tensors are packed back to back (256-byte aligned) into buckets of at most ``bucket_size``
bytes, in an order that lets the receiver finish one decoder layer after another (a layer's
fused weights can be rebuilt and its staging memory released as soon as its last projection
has arrived). A tensor larger than a bucket gets a bucket of its own; tensors marked
``direct`` skip the buckets and are received straight into the engine's storage. Tied
tensors (same storage under two names) travel once.
(reference: arctic_inference/server/weight_sync/schedule.py:54-146 for the assignment of
senders to targets; its bucket packing happens inside the engine, engine.py:86-169.)
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Iterable, Optional

import torch

ALIGN = 256
_DTYPES = {str(d).replace("torch.", ""): d for d in (
    torch.bfloat16, torch.float16, torch.float32, torch.float64, torch.int8, torch.uint8,
    torch.int32, torch.int64, torch.float8_e4m3fn, torch.float8_e5m2, torch.bool)}
_LAYER = re.compile(r"\.layers\.(\d+)\.")


def dtype_name(d: torch.dtype) -> str:
    return str(d).replace("torch.", "")


def dtype_from_name(s: str) -> torch.dtype:
    return _DTYPES[s]


@dataclass
class TensorMeta:
    name: str
    shape: tuple
    dtype: str
    direct: bool = False
    alias_of: Optional[str] = None      # tied to another tensor: not transferred

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * torch.empty(0, dtype=dtype_from_name(self.dtype)).element_size()

    @classmethod
    def of(cls, name: str, t: torch.Tensor, direct: bool = False) -> "TensorMeta":
        return cls(name, tuple(t.shape), dtype_name(t.dtype), direct)


@dataclass
class Slot:
    meta: TensorMeta
    offset: int


@dataclass
class Bucket:
    nbytes: int = 0
    slots: list = field(default_factory=list)


@dataclass
class TransferSchedule:
    buckets: list
    direct: list            # TensorMeta sent one by one
    aliases: list           # TensorMeta with alias_of set
    bucket_size: int

    @property
    def num_tensors(self) -> int:
        return sum(len(b.slots) for b in self.buckets) + len(self.direct)

    @property
    def total_bytes(self) -> int:
        return sum(s.meta.nbytes for b in self.buckets for s in b.slots) + \
            sum(m.nbytes for m in self.direct)

    @staticmethod
    def order_key(name: str):
        m = _LAYER.search(name)
        # embeddings / norms / heads first (they are independent), then layer by layer
        return (1, int(m.group(1)), name) if m else (0, 0, name)

    @classmethod
    def build(cls, metas: Iterable[TensorMeta] = (), bucket_size: int = 256 << 20, *more, **kw):
        """The bucket plan of ``metas``. Called the way the reference's class of this name is
        (``build(training_sharding, training_gpus, inference_replicas, inference_tp)``), it
        returns the :class:`SenderSchedule` of that deployment instead."""
        if isinstance(metas, str) or "training_sharding" in kw:
            args = ([metas, bucket_size] if isinstance(metas, str) else []) + list(more)
            return SenderSchedule.build(*args, **kw)
        metas = sorted(metas, key=lambda m: cls.order_key(m.name))
        buckets, direct, aliases = [], [], []
        cur = Bucket()
        for m in metas:
            if m.alias_of is not None:
                aliases.append(m)
                continue
            if m.direct:
                direct.append(m)
                continue
            need = (m.nbytes + ALIGN - 1) // ALIGN * ALIGN
            if cur.slots and cur.nbytes + need > bucket_size:
                buckets.append(cur)
                cur = Bucket()
            cur.slots.append(Slot(m, cur.nbytes))
            cur.nbytes += need
        if cur.slots:
            buckets.append(cur)
        return cls(buckets, direct, aliases, bucket_size)

    def max_bucket_bytes(self) -> int:
        return max([b.nbytes for b in self.buckets] + [0])

    # The plan crosses the wire as JSON text (never as pickled objects: the receiver must not
    # execute what a peer sends). Tensor entries use the field names of the reference's bucket
    # metadata, {"name", "shape", "dtype", "offset", "nbytes"}
    # (arctic_inference/server/weight_sync/engine.py:408-429).
    def to_json(self) -> str:
        import json

        def entry(m: TensorMeta, offset=None) -> dict:
            d = {"name": m.name, "shape": [int(x) for x in m.shape], "dtype": m.dtype,
                 "nbytes": m.nbytes}
            if offset is not None:
                d["offset"] = int(offset)
            if m.alias_of is not None:
                d["alias_of"] = m.alias_of
            return d

        return json.dumps({
            "version": 1, "bucket_size": int(self.bucket_size),
            "buckets": [{"nbytes": int(b.nbytes),
                         "tensors": [entry(s.meta, s.offset) for s in b.slots]}
                        for b in self.buckets],
            "direct": [entry(m) for m in self.direct],
            "aliases": [entry(m) for m in self.aliases]})

    @classmethod
    def from_json(cls, text) -> "TransferSchedule":
        """Parses and validates a plan received from a peer: known dtypes, non-negative
        sizes, slots inside their bucket, byte counts that match shape x dtype."""
        import json
        d = json.loads(text)
        if not isinstance(d, dict) or d.get("version") != 1:
            raise ValueError("weight stream: unknown plan format")

        def meta(e: dict, direct: bool = False) -> TensorMeta:
            if e["dtype"] not in _DTYPES:
                raise ValueError("weight stream: unknown dtype %r" % (e["dtype"],))
            shape = tuple(int(x) for x in e["shape"])
            if any(x < 0 for x in shape):
                raise ValueError("weight stream: negative dimension in %r" % (e["name"],))
            m = TensorMeta(str(e["name"]), shape, e["dtype"], direct, e.get("alias_of"))
            if int(e.get("nbytes", m.nbytes)) != m.nbytes:
                raise ValueError("weight stream: byte count of %r does not match its shape" % m.name)
            return m

        buckets = []
        for b in d["buckets"]:
            bk = Bucket(int(b["nbytes"]), [])
            for e in b["tensors"]:
                m = meta(e)
                off = int(e["offset"])
                if off < 0 or off % ALIGN or off + m.nbytes > bk.nbytes:
                    raise ValueError("weight stream: %r does not fit its bucket" % m.name)
                bk.slots.append(Slot(m, off))
            buckets.append(bk)
        return cls(buckets, [meta(e, True) for e in d["direct"]],
                   [meta(e) for e in d["aliases"]], int(d["bucket_size"]))


@dataclass
class TransferGroup:
    """One sending trainer rank and the serving ranks it feeds. Every (replica, tp_rank)
    target has its own two-party channel with the sender."""

    group_id: int
    sender_train_rank: int
    targets: list            # (replica_id, tp_rank) pairs

    WORLD_SIZE = 2

    @property
    def world_size(self) -> int:
        return self.WORLD_SIZE

    @property
    def replica_ids(self) -> list:
        return sorted({r for r, _ in self.targets})


@dataclass
class SenderSchedule:
    """Which trainer rank sends to which serving rank, fixed once per deployment. Serving rank
    ``(r, t)`` listens on ``base_port + r * inference_tp + t``.

    ``dp`` (every trainer rank holds the model) and ``fsdp`` (every rank ends up with each
    gathered parameter) use ``min(training_gpus, targets)`` senders and deal the targets out
    round-robin. ``zero3`` gathers parameters in a collective that every trainer rank must
    join, so every rank is a sender (possibly with no target) and, so that no sender walks the
    parameters twice while a gather is in flight, there must be at least as many trainer ranks
    as targets."""

    training_sharding: str
    training_gpus: int
    inference_replicas: int
    inference_tp: int
    groups: list = field(default_factory=list)

    @classmethod
    def build(cls, training_sharding: str, training_gpus: int, inference_replicas: int,
              inference_tp: int) -> "SenderSchedule":
        if training_sharding not in ("dp", "fsdp", "zero3"):
            raise ValueError("training_sharding must be 'dp', 'fsdp' or 'zero3', not %r"
                             % (training_sharding,))
        if min(training_gpus, inference_replicas, inference_tp) < 1:
            raise ValueError("training_gpus, inference_replicas and inference_tp must be >= 1")
        targets = [(r, t) for r in range(inference_replicas) for t in range(inference_tp)]
        if training_sharding == "zero3":
            if training_gpus < len(targets):
                raise ValueError("zero3 needs training_gpus (%d) >= inference_replicas * "
                                 "inference_tp (%d): one target per sender at most"
                                 % (training_gpus, len(targets)))
            senders = training_gpus
        else:
            senders = min(training_gpus, len(targets))
        dealt = [targets[i::senders] for i in range(senders)]
        return cls(training_sharding, training_gpus, inference_replicas, inference_tp,
                   [TransferGroup(i, i, t) for i, t in enumerate(dealt)])

    def port_for_target(self, replica_id: int, tp_rank: int, base_port: int) -> int:
        return base_port + replica_id * self.inference_tp + tp_rank

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    @property
    def active_sender_ranks(self) -> list:
        return [g.sender_train_rank for g in self.groups]

    def targets_of(self, train_rank: int) -> list:
        """(replica_id, tp_rank) pairs trainer rank ``train_rank`` sends to (possibly none)."""
        for g in self.groups:
            if g.sender_train_rank == train_rank:
                return list(g.targets)
        return []

    def ports_of(self, train_rank: int, base_port: int) -> list:
        return [self.port_for_target(r, t, base_port) for r, t in self.targets_of(train_rank)]


def find_aliases(named: dict) -> dict:
    """name -> first name that shares its storage (tied embeddings)."""
    seen, out = {}, {}
    for name, t in named.items():
        key = (t.data_ptr(), tuple(t.shape), t.dtype) if t.numel() else None
        if key is not None and key in seen:
            out[name] = seen[key]
        elif key is not None:
            seen[key] = name
    return out
