"""Result records returned by ``LLM.generate`` / streamed by the servers."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class CompletionOutput:
    index: int
    text: str
    token_ids: list[int]
    finish_reason: Optional[str] = None  # stop | length | abort
    logprobs: Optional[list] = None          # log-probability of every generated token
    cumulative_logprob: Optional[float] = None
    # per generated token, {token id: log-probability} of the most likely alternatives
    top_logprobs: Optional[list] = None


@dataclass
class RequestMetrics:
    arrival_time: float = 0.0
    first_scheduled_time: Optional[float] = None
    first_token_time: Optional[float] = None
    last_token_time: Optional[float] = None
    finished_time: Optional[float] = None
    num_cached_tokens: int = 0
    num_draft_tokens: int = 0
    num_accepted_tokens: int = 0

    @property
    def ttft(self) -> Optional[float]:
        if self.first_token_time is None:
            return None
        return self.first_token_time - self.arrival_time

    def tpot(self, num_output_tokens: int) -> Optional[float]:
        if self.finished_time is None or self.first_token_time is None or num_output_tokens < 2:
            return None
        return (self.finished_time - self.first_token_time) / (num_output_tokens - 1)


@dataclass
class RequestOutput:
    request_id: str
    prompt: Optional[str]
    prompt_token_ids: list[int]
    outputs: list[CompletionOutput]
    finished: bool
    metrics: RequestMetrics = field(default_factory=RequestMetrics)
    prompt_logprobs: Optional[list] = None
    num_cached_tokens: int = 0


@dataclass
class EmbeddingOutput:
    request_id: str
    embedding: list[float]
    prompt_token_ids: list[int]
