"""Same-node hand-over of a full set of weights without a network transfer.

A trainer that shares the machine (and usually the GPU) with the replica publishes its
tensors as IPC handles: CUDA tensors through CUDA IPC, host tensors through shared memory.
The handshake uses two small files under ``/dev/shm``:

    <key>.manifest   written by the sender: pickled {name: handle}; renamed into place
    <key>.done       written by the receiver once everything has been copied into the engine

The sender keeps the tensors alive until ``.done`` appears (bounded wait); the receiver maps
each tensor, feeds it to the same in-place updater as the network path, and unmaps it.
(reference: arctic_inference/server/weight_sync/ipc_engine.py:51-147,
receiver.py:443-567.)
"""

from __future__ import annotations

import os
import pickle
import time
from typing import Optional

import torch
from torch.multiprocessing.reductions import reduce_tensor

SHM_DIR = "/dev/shm"


def _paths(key: str, shm_dir: Optional[str] = None):
    base = os.path.join(shm_dir or SHM_DIR, "ab200_ws_" + key)
    return base + ".manifest", base + ".done"


def publish_ipc(named_tensors: dict, key: str, shm_dir: Optional[str] = None) -> str:
    """Sender: make ``named_tensors`` mappable by another process. The caller must keep the
    tensors alive until :func:`wait_ipc_done` returns."""
    manifest, done = _paths(key, shm_dir)
    if os.path.exists(done):
        os.remove(done)
    handles = {}
    for name, t in named_tensors.items():
        if not t.is_cuda:
            t.share_memory_()
        handles[name] = reduce_tensor(t.detach())
    tmp = manifest + ".tmp"
    with open(tmp, "wb") as f:
        pickle.dump(handles, f)
    os.replace(tmp, manifest)
    return manifest


def wait_ipc_done(key: str, timeout: float = 300.0, shm_dir: Optional[str] = None) -> dict:
    manifest, done = _paths(key, shm_dir)
    t0 = time.time()
    while not os.path.exists(done):
        if time.time() - t0 > timeout:
            raise TimeoutError("receiver did not finish the IPC weight update within %.0f s" % timeout)
        time.sleep(0.01)
    with open(done, "rb") as f:
        res = pickle.load(f)
    for p in (manifest, done):
        if os.path.exists(p):
            os.remove(p)
    return res


def open_ipc(key: str, timeout: float = 60.0, shm_dir: Optional[str] = None) -> dict:
    """Receiver: map the published tensors (name -> tensor sharing the sender's memory)."""
    manifest, _ = _paths(key, shm_dir)
    t0 = time.time()
    while not os.path.exists(manifest):
        if time.time() - t0 > timeout:
            raise TimeoutError("no IPC manifest %s after %.0f s" % (manifest, timeout))
        time.sleep(0.01)
    with open(manifest, "rb") as f:
        handles = pickle.load(f)
    return {name: fn(*args) for name, (fn, args) in handles.items()}


def finish_ipc(key: str, result: dict, shm_dir: Optional[str] = None) -> None:
    _, done = _paths(key, shm_dir)
    tmp = done + ".tmp"
    with open(tmp, "wb") as f:
        pickle.dump(result, f)
    os.replace(tmp, done)


def receive_ipc(engine, key: str, target: str = "model", shm_dir: Optional[str] = None) -> dict:
    t0 = time.time()
    tensors = open_ipc(key, shm_dir=shm_dir)
    try:
        if target == "speculator":
            from .receiver import _apply_speculator
            res = _apply_speculator(engine, iter(tensors.items()))
        else:
            from ...models.loader import LlamaWeightUpdater
            up = LlamaWeightUpdater(engine.runner.model)
            for name, t in tensors.items():
                up.deliver(name, t)
            res = up.finish()
        if engine.device.type == "cuda":
            torch.cuda.synchronize(engine.device)
    finally:
        tensors.clear()
    engine.reset_prefix_cache()
    res.update(direction="in", transport="ipc", seconds=time.time() - t0)
    rank = engine.comm.rank if engine.comm is not None else 0
    if rank == 0:
        finish_ipc(key, res, shm_dir)
    return res
