"""Per-request sampling controls (the subset of the vLLM-style surface the reference's
examples and tests use: README.md:126-158, tests/unit_tests/test_spec_dec_sleep.py:78-110;
``max_tokens_n`` is the rollout-replay extension of benchmark/rollout/sampling_params.patch)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    # penalties on tokens already generated (presence: once, frequency: per occurrence) and on
    # tokens of the prompt or the output (repetition: divides positive logits, multiplies
    # negative ones); logit_bias adds to the logits of the given token ids
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    logit_bias: Optional[dict] = None
    max_tokens: Optional[int] = 16
    min_tokens: int = 0
    ignore_eos: bool = False
    stop_token_ids: Optional[list[int]] = None
    stop: Optional[list[str]] = None
    include_stop_str_in_output: bool = False
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None
    seed: Optional[int] = None
    skip_special_tokens: bool = True
    # one forced length per parallel sample (len == n)
    max_tokens_n: Optional[list[int]] = None
    # structured output: the completion is exactly one of these strings / token-id lists
    guided_choice: Optional[list] = None
    # structured output: compact JSON conforming to this JSON schema (dict or JSON text)
    guided_json: Optional[object] = None
    # structured output: the whole completion matches this regular expression
    guided_regex: Optional[str] = None
    # or any matcher implementing structured.Grammar (one fresh object per request)
    grammar: Optional[object] = None
    extra_args: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.n < 1:
            raise ValueError("n must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
        if self.logit_bias:
            self.logit_bias = {int(k): float(v) for k, v in self.logit_bias.items()}
        if self.max_tokens is not None and self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.max_tokens_n is not None and len(self.max_tokens_n) != self.n:
            raise ValueError("max_tokens_n needs one entry per sample")
        if isinstance(self.stop, str):
            self.stop = [self.stop]

    @property
    def greedy(self) -> bool:
        return self.temperature <= 1e-5

    @property
    def needs_full_logits(self) -> bool:
        """True when arg-max / Gumbel-max over raw logits is not enough."""
        return (self.top_p < 1.0 or self.top_k > 0 or self.adjusts_logits or
                self.logprobs is not None or
                self.prompt_logprobs is not None or
                self.guided_choice is not None or self.guided_json is not None or
                self.guided_regex is not None or
                self.grammar is not None)

    @property
    def adjusts_logits(self) -> bool:
        return bool(self.min_p > 0.0 or self.presence_penalty or self.frequency_penalty or
                    self.repetition_penalty != 1.0 or self.logit_bias)

    def clone_for_sample(self, i: int) -> "SamplingParams":
        import copy
        sp = copy.copy(self)
        sp.n = 1
        sp.max_tokens_n = None
        if self.max_tokens_n is not None:
            sp.max_tokens = self.max_tokens_n[i]
        if self.seed is not None:
            sp.seed = self.seed + i
        return sp
