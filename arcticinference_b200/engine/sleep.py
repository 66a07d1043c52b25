"""Sleep / wake of an idle engine.

Level 1 releases the KV-cache tensors; level 2 additionally moves every weight
tensor (and the speculator's) to pinned host memory. Wake-up is staged by tags:
``["weights"]`` restores the weights (state WEIGHTS_READY, in which a weight sync
may overwrite them), ``["kv_cache"]`` re-creates the cache. Weight tensors are
restored *into their original device storage* when it still exists, so CUDA
graphs captured before the sleep stay valid.
(reference: arctic_inference/server/worker.py:275-390,
arctic_inference/vllm/patches.py:238-310)"""

from __future__ import annotations

import torch


def _model_tensors(engine):
    m = engine.runner.model
    items = [(m, "embed"), (m, "norm"), (m, "lm_head"), (m, "norm_swiftkv"), (m, "wkv_swiftkv")]
    for lw in m.layers:
        if lw is None:
            continue
        for name, _ in lw.tensors():
            items.append((lw, name))
        for key in list(lw.extra):
            items.append((lw.extra, key))
    prop = getattr(engine.runner, "proposer", None)
    if prop is not None and hasattr(prop, "weight_slots"):
        items.extend(prop.weight_slots())
    # an fp8 weight is two tensors (codes, block scales); its bf16 prefill shadow is derived
    # data, dropped while asleep and rebuilt on wake
    from ..models.quant import Fp8Weight
    out = []
    for owner, name in items:
        t = _get(owner, name) if (isinstance(owner, dict) and name in owner) or \
            (not isinstance(owner, dict) and hasattr(owner, name)) else None
        if isinstance(t, Fp8Weight):
            out.extend([(t, "q"), (t, "scale")])
        else:
            out.append((owner, name))
    return out


def mark_static_weights(engine) -> None:
    """Tell the linear layers which tensors are parameters (``ops.mark_static``)."""
    from .. import ops
    ops.clear_static()
    for owner, name in _model_tensors(engine):
        t = _get(owner, name) if (isinstance(owner, dict) and name in owner) or \
            (not isinstance(owner, dict) and hasattr(owner, name)) else None
        if isinstance(t, torch.Tensor) and t.is_cuda:
            ops.mark_static(t)


def _get(owner, name):
    return owner[name] if isinstance(owner, dict) else getattr(owner, name)


def _set(owner, name, value):
    if isinstance(owner, dict):
        owner[name] = value
    else:
        setattr(owner, name, value)


def sleep_engine(engine, level: int = 1) -> None:
    if level not in (1, 2):
        raise ValueError("sleep level must be 1 or 2")
    if engine.sleeping_level:
        return
    engine.kv_manager.reset_prefix_cache()
    engine.runner.kv.free()
    engine.runner._graphs.clear()
    prop = getattr(engine.runner, "proposer", None)
    if prop is not None and getattr(prop, "_graphs", None):
        prop._graphs.clear()       # its graphs hold the addresses of the weights
    engine._sleep_store = {}
    if level == 2:
        seen = {}
        from .. import ops
        from ..models.quant import Fp8Weight
        ops.clear_static()
        engine._sleep_shadows = []
        for owner, name in _model_tensors(engine):
            if isinstance(owner, Fp8Weight) and owner.shadow is not None:
                owner.shadow = None
                if owner not in engine._sleep_shadows:
                    engine._sleep_shadows.append(owner)
            t = _get(owner, name)
            if not isinstance(t, torch.Tensor) or not t.is_cuda:
                continue
            key = t.data_ptr()
            if key not in seen:
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                host.copy_(t)
                seen[key] = host
            engine._sleep_store[(id(owner), name)] = (owner, name, seen[key], t.device)
            _set(owner, name, None)
    if engine.device.type == "cuda":
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    engine.sleeping_level = level
    engine._awake_tags = set()


def wake_engine(engine, tags=None) -> None:
    if not engine.sleeping_level:
        return
    tags = set(tags) if tags is not None else {"weights", "kv_cache"}
    if "weights" in tags and "weights" not in engine._awake_tags:
        restored = {}
        for owner, name, host, dev in engine._sleep_store.values():
            if id(host) not in restored:
                restored[id(host)] = host.to(dev, non_blocking=True)
            _set(owner, name, restored[id(host)])
        engine._sleep_store = {}
        for w in getattr(engine, "_sleep_shadows", []):
            w.make_shadow()
        engine._sleep_shadows = []
        engine._awake_tags.add("weights")
        mark_static_weights(engine)
    if "kv_cache" in tags and "kv_cache" not in engine._awake_tags:
        engine.runner.init_kv_cache(engine.num_blocks)
        engine._awake_tags.add("kv_cache")
    if engine.device.type == "cuda":
        torch.cuda.synchronize()
    if engine.sleeping_level == 1:
        engine._awake_tags.add("weights")
    if {"weights", "kv_cache"} <= engine._awake_tags:
        engine.sleeping_level = 0
