"""Request state tracked by the scheduler."""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional

from .outputs import RequestMetrics
from .sampling_params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    PREEMPTED = 2
    FINISHED_STOPPED = 3
    FINISHED_LENGTH = 4
    FINISHED_ABORTED = 5

    @property
    def finished(self) -> bool:
        return self.value >= 3


_FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                  RequestStatus.FINISHED_ABORTED: "abort"}


@dataclass(eq=False)     # identity comparison: requests sit in lists that are searched every step
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    prompt: Optional[str] = None
    eos_token_id: Optional[int] = None
    extra_stop_ids: tuple = ()        # the model's further end-of-sequence ids (unless ignore_eos)
    parent_id: Optional[str] = None   # set for the samples of an n > 1 request
    sample_index: int = 0
    arrival_time: float = field(default_factory=time.time)
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    # number of tokens (prompt + output) whose KV is in the cache
    num_computed_tokens: int = 0
    block_ids: list[int] = field(default_factory=list)
    num_cached_tokens: int = 0
    # draft tokens to verify in the next step (speculative decoding)
    spec_token_ids: list[int] = field(default_factory=list)
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    output_logprobs: Optional[list] = None
    output_top_logprobs: Optional[list] = None
    prompt_logprobs: Optional[list] = None     # [None, log P(prompt[1] | prompt[:1]), ...]
    routing_key: Optional[str] = None
    _block_array: Optional[object] = field(default=None, repr=False)
    # run-ahead scheduling: the last output token is a placeholder for a token that has been
    # sampled on the device but not read yet / the request ends with that token whatever it is
    provisional: bool = False
    finishing: bool = False
    # run-ahead scheduling: tokens of a prompt chunk whose step is queued but not completed
    chunk_ahead: int = 0
    # structured output: matcher over the output tokens (structured.Grammar), advanced by
    # ``accept_output`` as tokens are appended
    grammar: Optional[object] = None
    # stop strings: matcher over the detokenised output (StopStringMatcher) and, once one was
    # found, the output text cut at it
    stop_matcher: Optional[object] = None
    stop_text: Optional[str] = None

    def __post_init__(self):
        self.metrics.arrival_time = self.arrival_time

    def block_array(self):
        """``block_ids`` as an int32 array, rebuilt only when the table grew (the KV manager
        drops it when it frees the request's blocks)."""
        a = self._block_array
        if a is None or a.size != len(self.block_ids):
            import numpy as np
            a = self._block_array = np.asarray(self.block_ids, dtype=np.int32)
        return a

    def tokens_slice(self, a: int, b: int) -> list:
        """Known tokens [a, b) without concatenating prompt and output."""
        n = len(self.prompt_token_ids)
        if b <= n:
            return self.prompt_token_ids[a:b]
        if a >= n:
            return self.output_token_ids[a - n:b - n]
        return self.prompt_token_ids[a:] + self.output_token_ids[:b - n]

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    @property
    def is_prefilling(self) -> bool:
        return self.num_computed_tokens < self.num_tokens - 1 or not self.output_token_ids and \
            self.num_computed_tokens < self.num_prompt_tokens

    @property
    def finish_reason(self) -> Optional[str]:
        return _FINISH_REASON.get(self.status)

    def check_stop(self, max_model_len: int) -> bool:
        """Update ``status`` after one token was appended; True when finished."""
        sp = self.sampling_params
        n_out = len(self.output_token_ids)
        if self.grammar is not None and n_out > 0:
            g = self.grammar
            if not g.finished:
                g.accept(self.output_token_ids[-1])
            if g.finished:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
        if n_out >= sp.min_tokens and n_out > 0:
            last = self.output_token_ids[-1]
            if not sp.ignore_eos and self.eos_token_id is not None and last == self.eos_token_id:
                self.status = RequestStatus.FINISHED_STOPPED
                return True
            if (sp.stop_token_ids and last in sp.stop_token_ids) or \
                    (self.extra_stop_ids and last in self.extra_stop_ids):
                self.status = RequestStatus.FINISHED_STOPPED
                return True
            if self.stop_matcher is not None and self.stop_matcher.hit(self):
                self.status = RequestStatus.FINISHED_STOPPED
                return True
        if (sp.max_tokens is not None and n_out >= sp.max_tokens) or \
                self.num_tokens >= max_model_len:
            self.status = RequestStatus.FINISHED_LENGTH
            return True
        return False


class StopStringMatcher:
    """Ends a request when its detokenised output contains one of ``stop`` strings; the text
    handed back is cut before the match (after it with ``include_stop_str_in_output``). The
    output is decoded again from the start at every token: stop strings are for interactive
    requests, whose outputs are short next to the cost of a model step."""

    def __init__(self, tokenizer, stop, include: bool = False, skip_special_tokens: bool = True):
        self.tokenizer = tokenizer
        self.stop = [s for s in ([stop] if isinstance(stop, str) else list(stop)) if s]
        self.include = include
        self.skip_special_tokens = skip_special_tokens

    def hit(self, req: "Request") -> bool:
        text = self.tokenizer.decode(req.output_token_ids,
                                     skip_special_tokens=self.skip_special_tokens)
        best = None
        for s in self.stop:
            i = text.find(s)
            if i >= 0 and (best is None or i < best[0]):
                best = (i, s)
        if best is None:
            return False
        req.stop_text = text[:best[0] + (len(best[1]) if self.include else 0)]
        return True
