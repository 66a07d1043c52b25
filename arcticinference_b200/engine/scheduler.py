"""Continuous-batching scheduler with chunked prefill and speculative placeholders.

Every step hands the model a flat token batch: each scheduled request
contributes the tokens whose KV is not in the cache yet (one token plus its
draft tokens in decode; a chunk of the prompt in prefill), within a token
budget. Decoding requests are scheduled first so that a long prompt cannot
starve them. When blocks run out the most recently admitted request is
preempted and recomputed later.

Draft handling follows the reference's scheduler hooks
(arctic_inference/vllm/patches.py:59-218): the width reserved for a request's
draft is what the proposer actually produced for it, requests beyond
``effective_draft_limit(batch)`` carry no draft, and after verification the
cache position advances only over accepted tokens.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..config import SchedulerConfig, SpeculativeConfig
from .kv_cache import KVCacheManager
from .request import Request, RequestStatus

PLACEHOLDER_TOKEN = -1      # same value as model_runner.PLACEHOLDER_TOKEN


@dataclass
class ScheduledRequest:
    request: Request
    start: int            # first position computed this step
    num_tokens: int       # tokens fed to the model (including draft tokens)
    num_draft: int        # trailing draft tokens among them
    samples: bool         # True if the step produces a new token for this request


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    total_tokens: int = 0
    preempted: list[Request] = field(default_factory=list)
    step_id: int = 0

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class Scheduler:
    def __init__(self, config: SchedulerConfig, kv: KVCacheManager,
                 spec: Optional[SpeculativeConfig] = None, token_multiple: int = 1):
        self.config = config
        self.kv = kv
        self.spec = spec
        # total tokens per step are padded by the runner to this multiple (SP size); the
        # budget is kept a multiple of it so padding never exceeds the budget
        self.token_multiple = token_multiple
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished: list[Request] = []
        self.step_id = 0

    # ------------------------------------------------------------------ queue management
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens >= self.config.max_model_len:
            raise ValueError("prompt (%d tokens) does not fit max_model_len=%d" %
                             (req.num_prompt_tokens, self.config.max_model_len))
        if req.num_prompt_tokens == 0:
            raise ValueError("empty prompt")
        self.waiting.append(req)

    def abort(self, request_id: str) -> Optional[Request]:
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.request_id == request_id:
                    q.remove(r)
                    r.status = RequestStatus.FINISHED_ABORTED
                    self.kv.free(r)
                    return r
        return None

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    def has_work(self) -> bool:
        return self.num_unfinished > 0

    # --------------------------------------------------------------------------- schedule
    def _preempt_last(self, out: SchedulerOutput, keep: Request) -> bool:
        for victim in reversed(self.running):
            if victim is keep:
                continue
            if any(s.request is victim for s in out.scheduled):
                continue
            self.running.remove(victim)
            self.kv.free(victim)
            victim.num_computed_tokens = 0
            victim.chunk_ahead = 0
            victim.spec_token_ids = []
            victim.status = RequestStatus.PREEMPTED
            self.waiting.appendleft(victim)
            out.preempted.append(victim)
            return True
        return False

    def schedule(self) -> SchedulerOutput:
        cfg = self.config
        out = SchedulerOutput(step_id=self.step_id)
        self.step_id += 1
        budget = cfg.max_num_batched_tokens // self.token_multiple * self.token_multiple
        now = time.time()

        # draft permission by position in the running batch
        decode_batch = sum(1 for r in self.running if not self._in_prefill(r))
        draft_limit = self.spec.effective_draft_limit(decode_batch) if self.spec else 0

        # 1) running requests (decodes and partially prefilled prompts)
        idx = 0
        bs = self.kv.block_size
        max_len = cfg.max_model_len
        sched_append = out.scheduled.append
        for req in list(self.running):
            if budget <= 0:
                break
            if out.preempted and req.status == RequestStatus.PREEMPTED:
                continue                 # preempted while serving an earlier request
            if req.finishing:
                continue                 # its last token is already on the way
            nt = len(req.prompt_token_ids) + len(req.output_token_ids)
            computed = req.num_computed_tokens
            prefilling = computed < nt - 1
            if not prefilling:
                # plain decode without a draft: one token, and usually no new block
                if not req.spec_token_ids and computed + 1 <= len(req.block_ids) * bs:
                    idx += 1
                    sched_append(ScheduledRequest(req, computed, 1, 0, True))
                    budget -= 1
                    continue
                if idx >= draft_limit:
                    req.spec_token_ids = []
                idx += 1
            else:
                req.spec_token_ids = []
            # never let a draft run past the model length
            room = max_len - nt - 1
            if len(req.spec_token_ids) > max(room, 0):
                req.spec_token_ids = req.spec_token_ids[:max(room, 0)]
            want = nt + len(req.spec_token_ids) - computed
            n = min(want, budget)
            if n < want and not cfg.enable_chunked_prefill and prefilling:
                continue
            if n < want:
                req.spec_token_ids = []  # a chunked prompt carries no draft
                n = min(nt - computed, budget)
            while not self.kv.can_allocate(req, n):
                if not self._preempt_last(out, req):
                    break
            if not self.kv.can_allocate(req, n):
                continue
            self.kv.allocate(req, n)
            nd = len(req.spec_token_ids)
            samples = computed + n >= nt + nd
            sched_append(ScheduledRequest(req, computed, n, nd if samples else 0, samples))
            budget -= n

        # 2) admit waiting requests
        while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs:
            req = self.waiting[0]
            if req.provisional:
                break   # preempted with a token still unread: re-admitted once it is known
            if req.num_computed_tokens == 0 and not req.block_ids:
                # every prompt position of a request that wants prompt log-probabilities has
                # to be computed, so it takes nothing from the prefix cache
                cached = self.kv.match_prefix(req) \
                    if req.sampling_params.prompt_logprobs is None else 0
                req.num_computed_tokens = cached
                req.num_cached_tokens = cached
                req.metrics.num_cached_tokens = cached
            want = req.num_tokens - req.num_computed_tokens
            n = min(want, budget)
            if n < want and not cfg.enable_chunked_prefill:
                break
            if not self.kv.can_allocate(req, n):
                if req.block_ids and req.num_computed_tokens == req.num_cached_tokens:
                    # give the cached prefix back; it is matched again when there is room
                    self.kv.free(req)
                    req.num_computed_tokens = 0
                break
            self.waiting.popleft()
            self.kv.allocate(req, n)
            req.status = RequestStatus.RUNNING
            if req.metrics.first_scheduled_time is None:
                req.metrics.first_scheduled_time = now
            self.running.append(req)
            samples = req.num_computed_tokens + n >= req.num_tokens
            out.scheduled.append(ScheduledRequest(req, req.num_computed_tokens, n, 0, samples))
            budget -= n

        out.total_tokens = sum(s.num_tokens for s in out.scheduled)
        return out

    @staticmethod
    def _in_prefill(req: Request) -> bool:
        return req.num_computed_tokens < req.num_tokens - 1

    # ----------------------------------------------------------------------------- run-ahead
    def advance_provisionally(self, out: SchedulerOutput) -> None:
        """Book the outcome of a step before the host has read its tokens, so that the next
        step can be scheduled and queued while this one still runs: a prompt chunk advances
        the request's computed position; a sampling request also receives a placeholder for
        the token it is about to get (``update_from_output`` puts the real one in). Draft
        verification cannot be booked ahead (the accepted length is unknown)."""
        cfg = self.config
        for s in out.scheduled:
            req = s.request
            if req.status.finished or req.status == RequestStatus.PREEMPTED:
                continue
            assert not req.provisional and not req.chunk_ahead and s.num_draft == 0
            req.num_computed_tokens += s.num_tokens
            if not s.samples:
                req.chunk_ahead = s.num_tokens
                continue
            req.output_token_ids.append(PLACEHOLDER_TOKEN)
            req.provisional = True
            sp = req.sampling_params
            if (sp.max_tokens is not None and len(req.output_token_ids) >= sp.max_tokens) or \
                    req.num_tokens >= cfg.max_model_len:
                req.finishing = True

    # ----------------------------------------------------------------------------- update
    def update_from_output(self, out: SchedulerOutput, new_tokens: dict[str, list[int]],
                           drafts: Optional[dict[str, list[int]]] = None) -> list[Request]:
        """``new_tokens[request_id]``: tokens produced by this step for requests with
        ``samples`` set -- the accepted draft tokens followed by one token sampled from the
        model. ``drafts``: proposals for the next step. Returns requests that finished."""
        now = time.time()
        done = []
        for s in out.scheduled:
            req = s.request
            provisional = req.provisional
            if provisional:
                # the step was booked ahead of time: put the real token where the placeholder is
                req.provisional = False
                toks = new_tokens.get(req.request_id, [])
                if toks and req.output_token_ids and req.output_token_ids[-1] == PLACEHOLDER_TOKEN:
                    req.output_token_ids[-1] = toks[0]
            if provisional and req.status == RequestStatus.PREEMPTED:
                # preempted while its token was in flight: the token is now known and may
                # end the request, which then must not be admitted again
                req.finishing = False
                if req.metrics.first_token_time is None:
                    req.metrics.first_token_time = now
                req.metrics.last_token_time = now
                if req.check_stop(self.config.max_model_len):
                    req.metrics.finished_time = now
                    self.waiting.remove(req)
                    self.kv.free(req)
                    self.finished.append(req)
                    done.append(req)
                else:
                    req.status = RequestStatus.PREEMPTED
                continue
            if req.status.finished or req.status == RequestStatus.PREEMPTED:
                continue
            if not s.samples:
                if req.chunk_ahead:
                    req.chunk_ahead = 0          # the position was advanced when it was booked
                else:
                    req.num_computed_tokens += s.num_tokens
                self.kv.commit(req, req.num_computed_tokens)
                continue
            toks = new_tokens.get(req.request_id, [])
            assert toks, "a sampling request must receive at least one token"
            if provisional:
                req.finishing = False
                if req.metrics.first_token_time is None:
                    req.metrics.first_token_time = now
                req.metrics.last_token_time = now
                finished = req.check_stop(self.config.max_model_len)
                self.kv.commit(req, min(req.num_computed_tokens, req.num_tokens))
                if finished:
                    req.metrics.finished_time = now
                    self.running.remove(req)
                    self.kv.free(req)
                    self.finished.append(req)
                    done.append(req)
                continue
            accepted = len(toks) - 1
            assert accepted <= s.num_draft
            # KV is valid for the fed tokens up to and including the accepted drafts
            req.num_computed_tokens += s.num_tokens - (s.num_draft - accepted)
            if s.num_draft:
                req.metrics.num_draft_tokens += s.num_draft
                req.metrics.num_accepted_tokens += accepted
            req.spec_token_ids = []
            if req.metrics.first_token_time is None:
                req.metrics.first_token_time = now
            finished = False
            for t in toks:
                req.output_token_ids.append(t)
                if req.check_stop(self.config.max_model_len):
                    finished = True
                    break
            req.metrics.last_token_time = now
            self.kv.commit(req, min(req.num_computed_tokens, req.num_tokens))
            if finished:
                req.metrics.finished_time = now
                self.running.remove(req)
                self.kv.free(req)
                self.finished.append(req)
                done.append(req)
            elif drafts:
                d = drafts.get(req.request_id)
                if d:
                    d = list(d)
                    if req.grammar is not None:
                        # a draft may only run as far as the grammar allows
                        d = d[:req.grammar.validate_draft(d)]
                    req.spec_token_ids = d
        return done
