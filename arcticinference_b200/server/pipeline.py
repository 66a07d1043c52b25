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
        return await self.fn(item, self.pipeline.handle)

    def __get__(self, obj, objtype=None):     # a task defined inside a class stays a plain attribute
        return self

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
                        results[i] = await self.fn(item, self.pipeline.handle)
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


class LLMHandle:
    """What a task function gets as its second argument. Called like a function it is this
    package's form, ``await llm(prompt, sampling_params, routing_key=...)`` -> result dict;
    ``generate`` / ``generate_token_ids`` are the reference's form
    (arctic_inference/server/pipeline.py:19-42): sampling parameters as keywords, the text or
    the token ids returned, ``retries`` further attempts one second apart."""

    def __init__(self, pipeline: "Pipeline", backend, model_id: Optional[str] = None):
        self._pipeline, self._backend, self._model_id = pipeline, backend, model_id

    async def __call__(self, prompt, sampling_params: Optional[dict] = None, routing_key=None,
                       strict: bool = False) -> dict:
        res = await self._backend.generate(prompt, sampling_params, model_id=self._model_id,
                                           routing_key=routing_key, strict=strict)
        return res[0]

    async def _retrying(self, prompt, key: str, retries: int, params: dict):
        for attempt in range(retries + 1):
            try:
                return (await self(prompt, params))[key]
            except asyncio.CancelledError:
                raise
            except Exception as e:  # noqa: BLE001 - retried
                if attempt == retries:
                    raise
                logger.warning("LLM call failed (attempt %d of %d): %s", attempt + 1, retries + 1, e)
                await asyncio.sleep(self._pipeline.retry_delay)

    async def generate(self, prompt: str, retries: int = 3, **sampling) -> str:
        return await self._retrying(prompt, "text", retries, sampling)

    async def generate_token_ids(self, prompt_token_ids: list, retries: int = 3, **sampling) -> list:
        return await self._retrying(list(prompt_token_ids), "token_ids", retries, sampling)


class Pipeline:
    """``Pipeline(pool)`` or ``Pipeline({"name": pool, ...})`` (the task then gets a dict of
    handles). Two ways to use it:

        @pipeline.task                       # the reference's: one task, run by the pipeline
        async def f(sample, llm): return await llm.generate(prompt=sample["text"], max_tokens=64)
        results = await pipeline.run(dataset)

        @pipeline.task(max_in_flight=256, retries=2)     # several tasks, each run on its own
        async def g(item, llm): return await llm(item["text"], {"max_tokens": 64})
        results = await g.run(dataset)
    """

    retry_delay = 1.0        # seconds between the attempts of LLMHandle.generate

    def __init__(self, backend, model_id: Optional[str] = None):
        self.backend = backend
        self.model_id = model_id
        if isinstance(backend, dict):
            if not backend:
                raise ValueError("pools must not be empty")
            self.handle = {name: LLMHandle(self, pool) for name, pool in backend.items()}
        else:
            self.handle = LLMHandle(self, backend, model_id)
        self._task: Optional[PipelineTask] = None

    async def run(self, dataset, max_retries: Optional[int] = None, show_progress: bool = False) -> list:
        """Run the task registered with ``@pipeline.task`` over ``dataset``; results in dataset
        order. An item that still fails after ``max_retries`` further attempts yields
        ``{"__error__": message}`` (``None``: keep retrying, at most 1000 times)."""
        if self._task is None:
            raise RuntimeError("no task registered: use @pipeline.task")
        t = PipelineTask(self, self._task.fn, self._task.max_in_flight,
                         1000 if max_retries is None else max_retries, return_exceptions=True)
        bar = None
        if show_progress:
            try:
                import tqdm
                bar = tqdm.tqdm(total=len(dataset), desc="Processing")
            except ImportError:
                bar = None
        try:
            res = await t.run(dataset, progress=(lambda done, n: bar.update(1)) if bar else None)
        finally:
            if bar is not None:
                bar.close()
        return [{"__error__": str(r.cause)} if isinstance(r, TaskError) else r for r in res]

    async def generate(self, prompt, sampling_params: Optional[dict] = None, routing_key=None,
                       strict: bool = False) -> dict:
        if isinstance(self.handle, dict):
            raise TypeError("a pipeline over several pools has one handle per pool")
        return await self.handle(prompt, sampling_params, routing_key=routing_key, strict=strict)

    def task(self, fn: Optional[Callable] = None, *, max_in_flight: int = MAX_IN_FLIGHT,
             retries: int = 2, return_exceptions: bool = False):
        def wrap(f):
            import inspect
            if not inspect.iscoroutinefunction(f):
                raise ValueError("a pipeline task must be an async function")
            if len(inspect.signature(f).parameters) != 2:
                raise ValueError("a pipeline task takes exactly two parameters (sample, llm)")
            self._task = PipelineTask(self, f, max_in_flight, retries, return_exceptions)
            return self._task
        return wrap(fn) if fn is not None else wrap
