"""Minimal safetensors reader / writer (no dependency on the ``safetensors`` package).

File format: 8-byte little-endian header length, a JSON header mapping tensor names to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian tensor bytes. The reader memory-maps the file, so
iterating a multi-gigabyte shard does not copy it.
(The reference reads only the header this way: arctic_inference/server/weight_sync/utils.py:119-143.)
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from typing import Iterator

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn,
    "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n))


def read_safetensors(path: str) -> Iterator:
    """Yield (name, tensor) pairs; tensors are views into a read-only memory map."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = _DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        if e == b:
            yield name, torch.empty(info["shape"], dtype=dt)
            continue
        raw = np.frombuffer(mm, dtype=np.uint8, count=e - b, offset=base + b)
        with warnings.catch_warnings():
            # the view is read-only on purpose (consumers copy into engine storage); torch
            # warns about every non-writable array it wraps
            warnings.simplefilter("ignore", UserWarning)
            t = torch.from_numpy(raw)
        yield name, t.view(dt).reshape(info["shape"])


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
