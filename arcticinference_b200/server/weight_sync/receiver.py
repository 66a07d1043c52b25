"""Receiving side of a weight update, executed inside a replica's engine.

The functions here run on the engine's own thread between two steps, on every rank of the
replica (``AsyncLLM.apply``), so an update never interleaves with a forward pass and each
rank fills its own shard from its own channel (port ``master_port + rank``):

* ``engine_weights_info``: what to send (checkpoint names, full shapes, dtype, whether a
  tensor is received straight into engine storage);
* ``engine_sync_weights``: connect to the sender, stream, apply in place, acknowledge;
  ``reverse=True`` streams the engine's weights to the peer instead; an ``ipc://key``
  address switches to the shared-memory hand-over of ``ipc_engine``;
* ``engine_close_weight_sync``: drop cached channels.

(reference: arctic_inference/server/weight_sync/receiver.py:196-331.)
"""

from __future__ import annotations

import time
from dataclasses import asdict

import torch

from .engine import Alias, Channel, ack, receive_stream, send_stream
from .schedule import TensorMeta, TransferSchedule, find_aliases
from .utils import expected_llama_tensors, export_llama_state


def _rank(engine) -> int:
    return engine.comm.rank if engine.comm is not None else 0


def engine_weights_info(engine) -> list:
    m = engine.runner.model
    return [asdict(t) for t in expected_llama_tensors(m.cfg, m.dtype)]


def engine_spec_weights_info(engine) -> list:
    prop = getattr(engine.runner, "proposer", None)
    if prop is None:
        return []
    from .schedule import dtype_name
    return [asdict(TensorMeta("speculator." + k, tuple(t.shape), dtype_name(t.dtype)))
            for k, t in sorted(prop.w.items())]


def _channels(engine) -> dict:
    if not hasattr(engine, "_weight_sync_channels"):
        engine._weight_sync_channels = {}
    return engine._weight_sync_channels


def _apply_speculator(engine, stream) -> dict:
    prop = engine.runner.proposer
    n = 0
    staged = []
    for name, t in stream:
        if isinstance(t, Alias) or t is None:
            continue
        staged.append((name, t.clone()))
        n += 1
    # reuse the checkpoint loader's name handling (prefix, split LSTM gates), then copy in place
    old = dict(prop.w)
    prop.load_state(staged)
    for k, dst in old.items():
        new = prop.w.get(k)
        if new is not None and new is not dst:
            if new.shape != dst.shape and getattr(prop, "tp_comm", None) is not None and \
                    k.startswith("head"):
                new = new[prop.tp_offset:prop.tp_offset + prop.tp_rows]   # this rank's vocabulary rows
            dst.copy_(new.to(dst.dtype))
            prop.w[k] = dst
    # the fp8 copies of the LM heads follow their (now updated) bf16 originals, in place
    for k, q in (getattr(prop, "qhead", None) or {}).items():
        if k in prop.w:
            q.requantize_from(prop.w[k])
    return {"tensors": n, "layers": 0, "incomplete_layers": []}


def engine_sync_weights(engine, kw: dict) -> dict:
    t0 = time.time()
    addr = kw.get("master_addr")
    target = kw.get("target", "model")
    if isinstance(addr, str) and addr.startswith("ipc://"):
        from .ipc_engine import receive_ipc
        return receive_ipc(engine, addr[len("ipc://"):], target)
    port = int(kw["master_port"]) + _rank(engine)
    dev = engine.device
    ch = Channel(addr, port, rank=1, device=dev, timeout=float(kw.get("timeout", 120.0)))
    _channels(engine)[(addr, port)] = ch
    try:
        if kw.get("reverse"):
            if target == "speculator":
                named = {"speculator." + k: t for k, t in engine.runner.proposer.w.items()}
            else:
                named = dict(export_llama_state(engine.runner.model))
            al = find_aliases(named)
            metas = [TensorMeta.of(n, t) for n, t in named.items()]
            for m in metas:
                m.alias_of = al.get(m.name)
            sched = TransferSchedule.build(metas, int(kw.get("bucket_size") or (256 << 20)))
            applied = send_stream(ch, named, sched)
            return {"direction": "out", "tensors": applied, "bytes": sched.total_bytes,
                    "seconds": time.time() - t0}
        if target == "speculator":
            res = _apply_speculator(engine, receive_stream(ch))
        else:
            from ...models.loader import LlamaWeightUpdater
            up = LlamaWeightUpdater(engine.runner.model)
            direct = (lambda m: up.direct_target(m.name)) if kw.get("direct_mode", True) else None
            for name, t in receive_stream(ch, direct):
                up.deliver(name, t)
            res = up.finish()
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        ack(ch, res["tensors"])
        if res["incomplete_layers"]:
            raise RuntimeError("weight update left layers %s incomplete" % res["incomplete_layers"][:8])
        if not kw.get("engine_only"):
            engine.reset_prefix_cache()
        res.update(direction="in", seconds=time.time() - t0, rank=_rank(engine))
        return res
    finally:
        ch.close()
        _channels(engine).pop((addr, port), None)


def engine_close_weight_sync(engine) -> dict:
    chans = _channels(engine)
    n = len(chans)
    for ch in chans.values():
        ch.close()
    chans.clear()
    return {"closed": n}
