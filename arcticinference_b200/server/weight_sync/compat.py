"""The weight-sync names a trainer written against the reference imports
(arctic_inference/server/weight_sync/__init__.py:15-48), on top of this package's channel and
stream: ``NCCLEngine`` (one two-party channel: rank 0 sends, rank 1 receives),
``WeightInfo`` / ``build_weights_info`` (names, shapes and dtypes read from safetensors
headers), ``load_spec_checkpoint`` / ``spec_bucket_size`` / ``send_spec_weights`` for
speculators, and the shared-memory hand-over under its reference names."""

from __future__ import annotations

import glob
import os
import time
from typing import Iterable, Iterator, Optional

import torch

from ...utils.safetensors_io import _DTYPES, read_header, read_safetensors
from .engine import Channel, ack, receive_stream, send_stream
from .ipc_engine import _paths, open_ipc, publish_ipc
from .schedule import TensorMeta, TransferSchedule, find_aliases

DEFAULT_BUCKET_SIZE = 256 << 20


class WeightInfo:
    """Name, shape and dtype of one checkpoint tensor."""

    __slots__ = ("name", "shape", "dtype")

    def __init__(self, name: str, shape, dtype: torch.dtype):
        self.name, self.shape, self.dtype = name, torch.Size(shape), dtype

    @property
    def nbytes(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n * torch.empty((), dtype=self.dtype).element_size()

    def to_dict(self) -> dict:
        return {"name": self.name, "shape": list(self.shape), "dtype": str(self.dtype)}

    @classmethod
    def from_dict(cls, d: dict) -> "WeightInfo":
        return cls(d["name"], d["shape"], getattr(torch, str(d["dtype"]).replace("torch.", "")))

    def __repr__(self) -> str:
        return "WeightInfo(%r, %s, %s)" % (self.name, tuple(self.shape), self.dtype)


def build_weights_info(model_path: str) -> list:
    """One :class:`WeightInfo` per tensor of a checkpoint directory, from the safetensors
    headers alone (no tensor data is read)."""
    files = sorted(glob.glob(os.path.join(model_path, "*.safetensors")))
    if not files:
        raise FileNotFoundError("no safetensors files in %s" % model_path)
    out = []
    for f in files:
        for name, info in read_header(f).items():
            if name != "__metadata__":
                out.append(WeightInfo(name, info["shape"], _DTYPES.get(info["dtype"], torch.float32)))
    return out


class NCCLEngine:
    """One two-party weight channel: rank 0 sends, rank 1 receives. The transport is NCCL
    when ``device`` is a GPU and gloo for host tensors. With ``reverse`` the receiver hosts
    the rendezvous (the TCP listener role is independent of who sends)."""

    def __init__(self, master_addr: str, master_port: int, rank: int, world_size: int = 2,
                 device=None, bucket_size: int = DEFAULT_BUCKET_SIZE, reverse: bool = False,
                 timeout: float = 300.0):
        if world_size != 2 or rank not in (0, 1):
            raise ValueError("a weight channel has exactly two parties (rank 0 sends, rank 1 receives)")
        self.rank, self.world_size, self.bucket_size = rank, world_size, bucket_size
        self.is_sender = rank == 0
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        # the channel's rank 0 hosts the store; with `reverse` that is the receiver
        self._ch = Channel(master_addr, master_port, rank=(1 - rank) if reverse else rank,
                           device=self.device, timeout=timeout)

    def send_weights(self, weights: Iterable) -> dict:
        """Stream ``(name, tensor)`` pairs to the receiver in buckets; returns statistics."""
        assert self.is_sender, "only rank 0 sends"
        t0 = time.time()
        named = dict(weights)
        al = find_aliases(named)
        metas = []
        for n, t in named.items():
            m = TensorMeta.of(n, t)
            m.alias_of = al.get(n)
            metas.append(m)
        sched = TransferSchedule.build(metas, self.bucket_size)
        applied = send_stream(self._ch, named, sched)
        dt = time.time() - t0
        return {"num_tensors": applied, "total_bytes": sched.total_bytes, "elapsed_s": dt,
                "num_buckets": len(sched.buckets)}

    def receive_weights(self) -> Iterator:
        """Yield ``(name, tensor)``; a bucketed tensor is a view that the next but one bucket
        overwrites, so use (copy) it before asking for more."""
        assert not self.is_sender, "rank 0 sends"
        n = 0
        for name, t in receive_stream(self._ch):
            n += 1
            yield name, t
        ack(self._ch, n)

    def destroy(self) -> None:
        self._ch.close()


def load_spec_checkpoint(path: str) -> dict:
    """Tensors of a speculator checkpoint directory (safetensors or ``pytorch_model.bin``),
    names without the ``speculator.`` prefix."""
    out = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        for f in files:
            out.update({n: t.clone() for n, t in read_safetensors(f)})
    else:
        for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
            out.update(torch.load(f, map_location="cpu", weights_only=True))
    if not out:
        raise FileNotFoundError("no speculator weights in %s" % path)
    return {(n[len("speculator."):] if n.startswith("speculator.") else n): t for n, t in out.items()}


def spec_bucket_size(weights: dict, limit: int = DEFAULT_BUCKET_SIZE) -> int:
    """A bucket that holds the largest speculator tensor (the vocabulary heads), capped."""
    biggest = max((t.numel() * t.element_size() for t in weights.values()), default=0)
    return max(1 << 20, min(limit, (biggest + 255) // 256 * 256))


def send_spec_weights(weights: dict, groups: list, device: Optional[str] = None, **kw) -> list:
    """Send a speculator's tensors to the replicas of ``groups`` (as ``WeightSender.send``)."""
    from .sender import WeightSender
    kw.setdefault("bucket_size", spec_bucket_size(weights))
    return WeightSender(weights, device=device or "cpu").send(groups, **kw)


# the shared-memory hand-over between a trainer and replicas on one node
def save_weights_to_shm(named_tensors: dict, key: str, shm_dir: Optional[str] = None) -> str:
    return publish_ipc(named_tensors, key, shm_dir)


def load_weights_from_shm(key: str, timeout: float = 60.0, shm_dir: Optional[str] = None) -> dict:
    return open_ipc(key, timeout, shm_dir)


def cleanup_shm(key: str, shm_dir: Optional[str] = None) -> None:
    for p in _paths(key, shm_dir):
        try:
            os.remove(p)
        except OSError:
            pass
