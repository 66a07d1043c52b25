"""Asynchronous, streaming front of the engine: the object the servers are built on.

A loop thread owns the engine. Callers (asyncio coroutines in any thread) hand it messages --
add a request, abort one, sleep, wake, reset the prefix cache -- and receive streamed
``RequestOutput`` objects back on their own event loop.

Multi-GPU engines are SPMD: every rank runs the same scheduler and must admit the same
requests at the same step. Rank 0 is the only rank with callers; at the top of every loop
iteration it broadcasts the batch of messages it is about to apply over a host-side (gloo)
group, and the other ranks (``run_follower``) apply the same batch before taking the same
step. That broadcast is the whole control plane: there is no per-step pickled scheduler output
as in the multiprocess executor behind the reference's worker
(arctic_inference/server/worker.py:117-228, :414-513).
"""

from __future__ import annotations

import asyncio
import queue
import threading
import time
import uuid
from typing import AsyncIterator, Optional

from ..config import EngineArgs
from .llm_engine import LLMEngine
from .outputs import RequestOutput
from .sampling_params import SamplingParams

IDLE_WAIT_S = 0.05


class EngineDeadError(RuntimeError):
    pass


class _Stream:
    __slots__ = ("loop", "queue")

    def __init__(self, loop):
        self.loop = loop
        self.queue: asyncio.Queue = asyncio.Queue()

    def put(self, item) -> None:
        self.loop.call_soon_threadsafe(self.queue.put_nowait, item)


class AsyncLLM:
    def __init__(self, engine: LLMEngine):
        self.engine = engine
        self.comm = engine.comm
        self.rank = self.comm.rank if self.comm is not None else 0
        self.world = self.comm.world if self.comm is not None else 1
        self._inbox: "queue.Queue" = queue.Queue()
        self._streams: dict[str, _Stream] = {}
        self._thread: Optional[threading.Thread] = None
        self._dead: Optional[BaseException] = None
        self._stopped = False
        self.paused = False

    @classmethod
    def from_engine_args(cls, args: EngineArgs, device=None, comm=None) -> "AsyncLLM":
        if comm is None and args.tensor_parallel_size * args.ulysses_sequence_parallel_size > 1:
            from ..parallel.comm import init_communicator
            comm = init_communicator(args.tensor_parallel_size,
                                     args.ulysses_sequence_parallel_size,
                                     backend=args.comm_backend)
            if device is None and comm.device is not None:
                device = str(comm.device)
        elif comm is None and args.pipeline_parallel_size > 1:
            from ..parallel.pipeline import init_pipeline
            comm = init_pipeline(args.pipeline_parallel_size, device)
            if device is None and comm.device is not None:
                device = str(comm.device)
        return cls(LLMEngine.from_engine_args(args, device=device, comm=comm))

    @property
    def is_leader(self) -> bool:
        return self.rank == 0

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "AsyncLLM":
        """Start the loop thread (rank 0). Other ranks call :meth:`run_follower` instead."""
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop, name="engine-loop", daemon=True)
            self._thread.start()
        return self

    def run_follower(self) -> None:
        """Blocks until rank 0 shuts the engine down."""
        assert not self.is_leader
        self._loop()

    def shutdown(self) -> None:
        if self._stopped:
            return
        self._stopped = True
        self._inbox.put(("shutdown",))
        if self._thread is not None:
            self._thread.join(timeout=30)

    # ------------------------------------------------------------------ the loop
    def _collect(self) -> list:
        """Messages to apply before the next step (rank 0): everything queued; when the
        engine is idle, wait briefly so that followers are not spun at full speed."""
        msgs = []
        block = not self.engine.has_unfinished_requests() or self.engine.sleeping_level
        try:
            msgs.append(self._inbox.get(timeout=IDLE_WAIT_S) if block else self._inbox.get_nowait())
            while True:
                msgs.append(self._inbox.get_nowait())
        except queue.Empty:
            pass
        return msgs

    def _loop(self) -> None:
        eng = self.engine
        futures = []
        try:
            if eng.device.type == "cuda":
                import torch
                # "cuda" without an index means the device that is current in the caller
                torch.cuda.set_device(eng.device if eng.device.index is not None
                                      else torch.cuda.current_device())
            while True:
                msgs = self._collect() if self.is_leader else None
                futures = []
                if self.is_leader:
                    # strip the caller-side handles before the batch crosses processes
                    wire = []
                    for m in msgs:
                        if m[0] == "call":
                            futures.append(m[3])
                            wire.append(("call", m[1], m[2]))
                        else:
                            wire.append(m)
                    msgs = wire
                if self.world > 1:
                    msgs = self.comm.host_broadcast(msgs, src=0)
                stop = False
                fi = 0
                for m in msgs:
                    kind = m[0]
                    if kind == "add":
                        _, rid, ids, params, arrival, key = m
                        try:
                            eng.add_request(rid, ids, params, arrival_time=arrival, routing_key=key)
                        except Exception as e:  # noqa: BLE001 - reported to the caller
                            self._finish_stream(rid, e)
                    elif kind == "abort":
                        eng.abort_request(m[1])
                        self._finish_stream(m[1], None)
                    elif kind == "call":
                        res, err = None, None
                        try:
                            res = self._apply_call(m[1], m[2])
                        except Exception as e:  # noqa: BLE001
                            err = e
                        if self.is_leader:
                            fut = futures[fi]
                            fi += 1
                            fut[0].call_soon_threadsafe(_resolve, fut[1], res, err)
                    elif kind == "shutdown":
                        stop = True
                if stop:
                    break
                if eng.sleeping_level or not eng.has_unfinished_requests():
                    continue
                for ro in eng.step(partial=True):
                    st = self._streams.get(ro.request_id)
                    if st is None:
                        continue
                    st.put(ro)
                    if ro.finished:
                        del self._streams[ro.request_id]
        except BaseException as e:  # noqa: BLE001 - every waiter must learn of it
            self._dead = e
            dead = EngineDeadError("engine loop died: %r" % (e,))
            for rid in list(self._streams):
                self._finish_stream(rid, dead)
            # control calls of the batch in hand, and any still queued, fail as well
            for fut in futures:
                fut[0].call_soon_threadsafe(_resolve, fut[1], None, dead)
            while True:
                try:
                    m = self._inbox.get_nowait()
                except queue.Empty:
                    break
                if m[0] == "call":
                    m[3][0].call_soon_threadsafe(_resolve, m[3][1], None, dead)
            raise
        finally:
            for rid in list(self._streams):
                self._finish_stream(rid, EngineDeadError("engine shut down"))

    def _apply_call(self, name: str, args: tuple):
        eng = self.engine
        if name == "sleep":
            if eng.has_unfinished_requests():
                raise RuntimeError("cannot sleep with unfinished requests")
            eng.sleep(*args)
        elif name == "wake_up":
            eng.wake_up(*args)
        elif name == "reset_prefix_cache":
            eng.reset_prefix_cache()
        elif name == "stats":
            return eng.get_stats()
        elif name == "apply":
            fn, fargs = args
            return fn(eng, *fargs)
        else:
            raise ValueError("unknown engine call %r" % name)
        return None

    def _finish_stream(self, rid: str, err) -> None:
        st = self._streams.pop(rid, None)
        if st is not None:
            st.put(err if err is not None else _ABORTED)

    # ------------------------------------------------------------------ caller side
    def _check(self) -> None:
        if self._dead is not None:
            raise EngineDeadError("engine loop died: %r" % (self._dead,))
        if self._stopped:
            raise EngineDeadError("engine shut down")
        if not self.is_leader:
            raise RuntimeError("only rank 0 accepts requests")

    async def generate(self, prompt, sampling_params: Optional[SamplingParams] = None,
                       request_id: Optional[str] = None,
                       routing_key=None) -> AsyncIterator[RequestOutput]:
        """Stream of outputs of one request; the last one has ``finished = True``. Cancelling
        the consumer aborts the request."""
        self._check()
        if self.paused:
            raise RuntimeError("engine is paused")
        params = sampling_params or SamplingParams()
        rid = request_id or uuid.uuid4().hex
        tok = self.engine.tokenizer
        if isinstance(prompt, str):
            ids = tok.encode(prompt)
        elif isinstance(prompt, dict):
            ids = prompt.get("prompt_token_ids")
            if ids is None:
                ids = tok.encode(prompt["prompt"])
        else:
            ids = list(prompt)
        st = _Stream(asyncio.get_running_loop())
        self._streams[rid] = st
        self._inbox.put(("add", rid, [int(t) for t in ids], params, time.time(), routing_key))
        if self._dead is not None:      # the loop died between the check above and the put
            self._finish_stream(rid, EngineDeadError("engine loop died: %r" % (self._dead,)))
        try:
            while True:
                item = await st.queue.get()
                if item is _ABORTED:
                    return
                if isinstance(item, BaseException):
                    raise item
                yield item
                if item.finished:
                    return
        finally:
            if rid in self._streams:
                self._inbox.put(("abort", rid))

    async def generate_final(self, prompt, sampling_params=None, request_id=None,
                             routing_key=None) -> Optional[RequestOutput]:
        last = None
        async for out in self.generate(prompt, sampling_params, request_id, routing_key):
            last = out
        return last

    async def abort(self, request_id: str) -> None:
        self._check()
        self._inbox.put(("abort", request_id))

    async def _call(self, name: str, *args):
        self._check()
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        self._inbox.put(("call", name, args, (loop, fut)))
        return await fut

    async def sleep(self, level: int = 1) -> None:
        await self._call("sleep", level)

    async def wake_up(self, tags=None) -> None:
        await self._call("wake_up", tags)

    async def reset_prefix_cache(self) -> None:
        await self._call("reset_prefix_cache")

    async def get_stats(self) -> dict:
        return await self._call("stats")

    async def apply(self, fn, *args):
        """Run ``fn(engine, *args)`` on every rank's loop thread between two steps (weight
        updates and the like). ``fn`` and ``args`` must pickle when the engine spans several
        GPUs. Returns rank 0's result."""
        return await self._call("apply", fn, args)

    @property
    def num_unfinished(self) -> int:
        return len(self._streams)


class _Aborted:
    pass


_ABORTED = _Aborted()


def _resolve(fut, res, err) -> None:
    if fut.done():
        return
    if err is not None:
        fut.set_exception(err)
    else:
        fut.set_result(res)
