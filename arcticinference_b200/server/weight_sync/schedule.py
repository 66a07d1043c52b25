"""Transfer plan: which tensor travels in which bucket at which offset.

Tensors are packed back to back (256-byte aligned) into buckets of at most ``bucket_size``
bytes, in an order that lets the receiver finish one decoder layer after another (a layer's
fused weights can be rebuilt and its staging memory released as soon as its last projection
has arrived). A tensor larger than a bucket gets a bucket of its own; tensors marked
``direct`` skip the buckets and are received straight into the engine's storage. Tied
tensors (same storage under two names) travel once.
(reference: arctic_inference/server/weight_sync/schedule.py:54-146.)
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
    def build(cls, metas: Iterable[TensorMeta], bucket_size: int = 256 << 20) -> "TransferSchedule":
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
