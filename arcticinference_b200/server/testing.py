"""CPU-only stand-in for an inference worker: deterministic outputs, no model.

Lets the scheduler, the pool, the REST API and the pipeline be exercised without a GPU
(reference: arctic_inference/server/testing.py:1-134). The "completion" of a prompt is a
function of the prompt's tokens only, so that tests can predict it.
"""

from __future__ import annotations

import asyncio
import hashlib
from typing import Any, Optional

from .worker import WorkerBase, WorkerStatus


def dummy_tokens(prompt, n: int) -> list[int]:
    seed = hashlib.sha256(repr(prompt).encode()).digest()
    return [seed[i % 32] + 256 * (i // 32) for i in range(n)]


class DummyWorker(WorkerBase):
    def __init__(self, idx: int = 0, latency: float = 0.0, kv_per_request: float = 0.01,
                 fail_after: Optional[int] = None):
        super().__init__(idx)
        self.latency = latency
        self.kv_per_request = kv_per_request
        self.fail_after = fail_after
        self.calls = 0
        self.active = 0
        self.seen: list = []
        self.weights_version = 0
        self._cancel = asyncio.Event()
        self.prefix_seen: set = set()

    async def initialize(self, config) -> None:
        self.config = config
        self.status = WorkerStatus.READY

    async def generate(self, prompt, sampling_params: Optional[dict] = None,
                       request_id: Optional[str] = None, routing_key=None) -> dict[str, Any]:
        if self.status is not WorkerStatus.READY:
            raise RuntimeError("worker %d is %s" % (self.idx, self.status.value))
        self.calls += 1
        if self.fail_after is not None and self.calls > self.fail_after:
            raise ConnectionError("worker %d is gone" % self.idx)
        sp = sampling_params or {}
        n_out = int(sp.get("max_tokens", 16))
        self.active += 1
        self.seen.append(prompt)
        try:
            if self.latency:
                waiter = asyncio.ensure_future(self._cancel.wait())
                done, _ = await asyncio.wait([waiter], timeout=self.latency)
                if done:
                    raise RuntimeError("request cancelled")
                waiter.cancel()
            toks = dummy_tokens(prompt, n_out)
            plen = len(prompt) if not isinstance(prompt, str) else len(prompt.split())
            key = repr(prompt)[:64]
            cached = plen if key in self.prefix_seen else 0
            self.prefix_seen.add(key)
            out = {"text": " ".join(map(str, toks)), "token_ids": toks, "finish_reason": "length",
                   "prompt_len": plen, "generation_len": n_out, "prefix_cache_len": cached}
            if sp.get("logprobs") is not None:
                out["logprobs"] = [-(t % 7) / 7.0 for t in toks]
            if sp.get("prompt_logprobs") is not None:
                out["prompt_logprobs"] = [None] + [-0.5] * max(plen - 1, 0)
            return out
        finally:
            self.active -= 1

    async def cancel_inflight(self) -> int:
        n = self.active
        self._cancel.set()
        await asyncio.sleep(0)
        self._cancel = asyncio.Event()
        return n

    async def get_stats(self) -> dict:
        return {"running": self.active, "waiting": 0,
                "kv_cache_usage": min(1.0, self.active * self.kv_per_request),
                "prompt_tokens": 0, "generation_tokens": 0}

    async def sleep(self, level: int = 1) -> None:
        self.status = WorkerStatus.SLEEPING

    async def wake_up(self, tags=None) -> None:
        tags = set(tags) if tags else {"weights", "kv_cache"}
        self._awake = getattr(self, "_awake", set()) | tags
        if "kv_cache" in self._awake:
            self.status = WorkerStatus.READY
            self._awake = set()
        else:
            self.status = WorkerStatus.WEIGHTS_READY

    async def reset_prefix_cache(self) -> None:
        self.prefix_seen.clear()

    async def weights_info(self) -> list[dict]:
        return [{"name": "w", "shape": [4, 4], "dtype": "bfloat16"}]

    async def sync_weights(self, **kw) -> dict:
        self.weights_version += 1
        return {"worker": self.idx, "version": self.weights_version, "tensors": 1}

    async def shutdown(self) -> None:
        self.status = WorkerStatus.UNINITIALIZED
