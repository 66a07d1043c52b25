"""Dataset pipelines on top of a pool: ``@pipeline.task`` turns an async function of one item
into a runner over a whole dataset with bounded concurrency and retries.

    pipe = Pipeline(pool)

    @pipe.task(max_in_flight=256, retries=2)
    async def answer(item, generate):
        out = await generate(item["prompt"], {"max_tokens": 64})
        return {"id": item["id"], "text": out["text"]}

    results = await answer.run(dataset)        # same order as the dataset

(reference: arctic_inference/server/pipeline.py:44-156; at most 1024 items in flight.)
"""

from __future__ import annotations

import asyncio
import logging
from typing import Awaitable, Callable, Iterable, Optional

logger = logging.getLogger(__name__)

MAX_IN_FLIGHT = 1024


class TaskError(RuntimeError):
    def __init__(self, index: int, cause: BaseException):
        super().__init__("item %d failed: %s" % (index, cause))
        self.index = index
        self.cause = cause


class PipelineTask:
    def __init__(self, pipeline: "Pipeline", fn: Callable[..., Awaitable], max_in_flight: int,
                 retries: int, return_exceptions: bool):
        self.pipeline = pipeline
        self.fn = fn
        self.max_in_flight = max(1, min(max_in_flight, MAX_IN_FLIGHT))
        self.retries = retries
        self.return_exceptions = return_exceptions
        self.attempts = 0
        self.__name__ = getattr(fn, "__name__", "task")

    async def __call__(self, item):
        return await self.fn(item, self.pipeline.generate)

    async def run(self, dataset: Iterable, progress: Optional[Callable[[int, int], None]] = None) -> list:
        items = list(dataset)
        results: list = [None] * len(items)
        sem = asyncio.Semaphore(self.max_in_flight)
        done = 0

        async def one(i: int, item) -> None:
            nonlocal done
            async with sem:
                err: Optional[BaseException] = None
                for attempt in range(self.retries + 1):
                    self.attempts += 1
                    try:
                        results[i] = await self.fn(item, self.pipeline.generate)
                        err = None
                        break
                    except asyncio.CancelledError:
                        raise
                    except Exception as e:  # noqa: BLE001 - retried
                        err = e
                        logger.info("%s item %d attempt %d failed: %s", self.__name__, i, attempt + 1, e)
                        await asyncio.sleep(min(0.05 * 2 ** attempt, 1.0))
                if err is not None:
                    if not self.return_exceptions:
                        raise TaskError(i, err)
                    results[i] = TaskError(i, err)
                done += 1
                if progress is not None:
                    progress(done, len(items))

        tasks = [asyncio.ensure_future(one(i, it)) for i, it in enumerate(items)]
        try:
            await asyncio.gather(*tasks)
        except BaseException:
            for t in tasks:
                t.cancel()
            await asyncio.gather(*tasks, return_exceptions=True)
            raise
        return results


class Pipeline:
    def __init__(self, backend, model_id: Optional[str] = None):
        self.backend = backend
        self.model_id = model_id

    async def generate(self, prompt, sampling_params: Optional[dict] = None, routing_key=None,
                       strict: bool = False) -> dict:
        res = await self.backend.generate(prompt, sampling_params, model_id=self.model_id,
                                          routing_key=routing_key, strict=strict)
        return res[0]

    def task(self, fn: Optional[Callable] = None, *, max_in_flight: int = MAX_IN_FLIGHT,
             retries: int = 2, return_exceptions: bool = False):
        def wrap(f):
            return PipelineTask(self, f, max_in_flight, retries, return_exceptions)
        return wrap(fn) if fn is not None else wrap
