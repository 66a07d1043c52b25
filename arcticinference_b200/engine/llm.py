"""Offline entry point with the vLLM-style surface the reference documents
(README.md:126-158): ``LLM(model=..., ulysses_sequence_parallel_size=...,
enable_shift_parallel=..., speculative_config={...})``, ``generate``, ``chat``,
``sleep`` / ``wake_up``."""

from __future__ import annotations

import dataclasses
from typing import Optional, Sequence, Union

from ..config import EngineArgs
from .llm_engine import LLMEngine
from .outputs import RequestOutput
from .sampling_params import SamplingParams


class LLM:
    def __init__(self, model: str = "llama-tiny", device: Optional[str] = None, comm=None,
                 **kwargs):
        names = {f.name for f in dataclasses.fields(EngineArgs)}
        unknown = set(kwargs) - names
        if unknown:
            raise TypeError("unknown LLM arguments: %s" % sorted(unknown))
        self.engine_args = EngineArgs(model=model, **kwargs)
        if comm is None and self.engine_args.tensor_parallel_size * \
                self.engine_args.ulysses_sequence_parallel_size > 1:
            from ..parallel.comm import init_communicator
            comm = init_communicator(self.engine_args.tensor_parallel_size,
                                     self.engine_args.ulysses_sequence_parallel_size,
                                     backend=self.engine_args.comm_backend)
            if device is None and comm.device is not None:
                device = str(comm.device)
        elif comm is None and self.engine_args.pipeline_parallel_size > 1:
            from ..parallel.pipeline import init_pipeline
            comm = init_pipeline(self.engine_args.pipeline_parallel_size, device)
            if device is None and comm.device is not None:
                device = str(comm.device)
        self.engine = LLMEngine.from_engine_args(self.engine_args, device=device, comm=comm)

    def get_tokenizer(self):
        return self.engine.tokenizer

    def generate(self, prompts, sampling_params: Union[SamplingParams, Sequence[SamplingParams],
                                                       None] = None,
                 use_tqdm: bool = False) -> list[RequestOutput]:
        if isinstance(prompts, (str, dict)) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        if sampling_params is None:
            sampling_params = SamplingParams()
        ids = []
        for i, p in enumerate(prompts):
            sp = sampling_params[i] if isinstance(sampling_params, (list, tuple)) else sampling_params
            ids.append(self.engine.add_request(None, p, sp))
        done: dict[str, RequestOutput] = {}
        while self.engine.has_unfinished_requests():
            for ro in self.engine.step():
                done[ro.request_id] = ro
        return [done[i] for i in ids]

    def chat(self, messages, sampling_params: Optional[SamplingParams] = None, **kw):
        if messages and isinstance(messages[0], dict):
            messages = [messages]
        from ..utils.tokenizer import chat_token_ids
        tok = self.engine.tokenizer
        prompts = [{"prompt_token_ids": chat_token_ids(tok, m)} for m in messages]
        return self.generate(prompts, sampling_params)

    def sleep(self, level: int = 1) -> None:
        self.engine.sleep(level)

    def wake_up(self, tags=None) -> None:
        self.engine.wake_up(tags)

    def reset_prefix_cache(self) -> None:
        self.engine.reset_prefix_cache()
