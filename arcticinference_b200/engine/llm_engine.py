"""The engine: scheduler + KV manager + model runner behind ``add_request`` / ``step``.

One engine object runs in every rank's process (SPMD); request admission must
therefore be identical on every rank (offline ``LLM.generate`` calls are; the
servers broadcast admitted requests from rank 0 before each step).
"""

from __future__ import annotations

import os
import time
from typing import Iterable, Optional

import torch

from ..config import EngineArgs, EngineConfig
from ..utils.tokenizer import get_tokenizer
from .kv_cache import KVCacheManager
from .model_runner import ModelRunner
from .outputs import CompletionOutput, RequestOutput
from .request import Request, StopStringMatcher
from .sampling_params import SamplingParams
from .scheduler import Scheduler


def tp_rows_per_request(spec) -> int:
    """Upper bound of the rows one request can contribute to a tensor-parallel stretch of a
    sequence-parallel step: its sampled row plus one per draft token under verification."""
    return 1 + (spec.max_draft_tokens if spec is not None else 0)


class LLMEngine:
    def __init__(self, config: EngineConfig, device: Optional[str] = None, comm=None):
        self.config = config
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        shard = None
        if comm is not None:
            shard = comm.shard_spec()
        self.comm = comm
        self.runner = ModelRunner(config, self.device, comm=comm, shard=shard)
        if comm is not None and getattr(comm, "fused", False):
            m = self.runner.model
            sp = config.parallel.sp
            max_tokens = (config.scheduler.max_num_batched_tokens + sp - 1) // sp * sp + sp
            # largest step that runs tensor-parallel: with sequence parallelism only steps up
            # to the shift threshold and the sampled rows of SwiftKV's later layers do (one
            # row per request plus one per draft token, and a hybrid suffix draft can be as
            # long as the suffix tree is deep)
            max_tp = max_tokens
            if sp > 1:
                max_tp = min(max_tokens, max(config.parallel.shift_parallel_threshold,
                                             tp_rows_per_request(config.speculative) *
                                             config.scheduler.max_num_seqs) + sp)
            comm.setup(max_tokens, max_tp, m.blk_rows, config.model.hidden_size,
                       sp * m.h * m.D, swiftkv=config.model.is_swiftkv)
        self.runner.load_model()
        self.num_blocks = self.runner.determine_num_blocks()
        if self.runner.pp is not None:
            # the stages hold different amounts of weights; their schedulers must see one pool size
            self.num_blocks = self.runner.pp.min_over_stages(self.num_blocks, self.device)
        self.runner.init_kv_cache(self.num_blocks)
        self.kv_manager = KVCacheManager(self.num_blocks, config.cache.block_size,
                                         config.cache.enable_prefix_caching)
        self.scheduler = Scheduler(config.scheduler, self.kv_manager, config.speculative,
                                   token_multiple=config.parallel.sp)
        self.tokenizer = get_tokenizer(config.tokenizer or config.model.name_or_path,
                                       config.model.vocab_size)
        self._seq = 0
        self._pending = None            # a step queued on the device whose tokens are unread
        self._parents: dict[str, dict] = {}
        self.step_count = 0
        self.sleeping_level = 0
        self.stats = {"prompt_tokens": 0, "generation_tokens": 0, "steps": 0,
                      "draft_tokens": 0, "accepted_tokens": 0, "run_ahead_steps": 0,
                      # speculation by draft position: how often position i was drafted /
                      # accepted (drafts vary in width from request to request and step to
                      # step; reference: arctic_inference/vllm/stats.py:25-67)
                      "drafted_per_position": [], "accepted_per_position": [],
                      # steps per execution mode and device-side wait limits that ran out
                      "sp_steps": 0, "tp_steps": 0, "comm_timeouts": 0,
                      # host seconds per phase: scheduling, building + queueing a step, waiting
                      # for its tokens (the only phase the device is waited for), bookkeeping
                      "t_schedule": 0.0, "t_launch": 0.0, "t_wait": 0.0, "t_update": 0.0}
        if config.speculative is not None:
            from ..spec_decode.propose import attach_speculation
            attach_speculation(self)
        if self.device.type == "cuda":
            from .sleep import mark_static_weights
            mark_static_weights(self)
        # The objects built so far (weights' wrappers, graphs, tables) live as long as the
        # engine: take them out of the cyclic collector's generations, so that a full
        # collection during serving does not walk them. With several ranks stepping in lockstep
        # a long collection on one rank stalls all of them.
        if os.environ.get("AB200_GC_FREEZE", "1") != "0":
            import gc
            gc.collect()
            gc.freeze()

    @classmethod
    def from_engine_args(cls, args: EngineArgs, device=None, comm=None) -> "LLMEngine":
        return cls(args.create_engine_config(), device=device, comm=comm)

    # --------------------------------------------------------------- requests
    def add_request(self, request_id: Optional[str], prompt, params: SamplingParams,
                    arrival_time: Optional[float] = None, routing_key=None) -> str:
        if request_id is None:
            request_id = "req-%d" % self._seq
        self._seq += 1
        if self.runner.pp is not None and (params.logprobs is not None or
                                           params.prompt_logprobs is not None):
            raise NotImplementedError("log-probabilities with pipeline parallelism (the logits "
                                      "exist on the last stage only)")
        text = None
        if isinstance(prompt, str):
            text = prompt
            ids = self.tokenizer.encode(prompt)
        elif isinstance(prompt, dict):
            text = prompt.get("prompt")
            ids = prompt.get("prompt_token_ids")
            if ids is None:
                ids = self.tokenizer.encode(text)
        else:
            ids = list(prompt)
        if not (isinstance(ids, list) and all(type(t) is int for t in ids)):
            ids = [int(t) for t in ids]
        eos = self.config.model.eos_token_id
        if eos is None:
            eos = getattr(self.tokenizer, "eos_token_id", None)
        extra = () if params.ignore_eos else self.config.model.extra_eos_token_ids
        if params.prompt_logprobs is not None and self.config.model.is_swiftkv:
            raise ValueError("prompt_logprobs is not available for SwiftKV models: their later "
                             "layers run on the sampled rows only")
        now = arrival_time if arrival_time is not None else time.time()

        def stops():
            if not params.stop:
                return None
            return StopStringMatcher(self.tokenizer, params.stop,
                                     getattr(params, "include_stop_str_in_output", False),
                                     params.skip_special_tokens)

        if params.n == 1:
            self.scheduler.add_request(Request(request_id, ids, params, prompt=text,
                                               eos_token_id=eos, extra_stop_ids=extra,
                                               arrival_time=now,
                                               routing_key=routing_key,
                                               grammar=self._grammar_for(params, eos),
                                               stop_matcher=stops()))
        else:
            self._parents[request_id] = {"n": params.n, "done": {}, "prompt": text, "ids": ids}
            for i in range(params.n):
                self.scheduler.add_request(Request(
                    "%s#%d" % (request_id, i), ids, params.clone_for_sample(i), prompt=text,
                    eos_token_id=eos, extra_stop_ids=extra, parent_id=request_id, sample_index=i,
                    arrival_time=now,
                    grammar=self._grammar_for(params, eos, copy_given=True),
                    stop_matcher=stops()))
        return request_id

    def _grammar_for(self, params: SamplingParams, eos, copy_given: bool = False):
        """A fresh matcher for one sequence, or None when the request is unconstrained."""
        if params.guided_choice is None and params.guided_json is None and \
                params.guided_regex is None and params.grammar is None:
            return None
        from ..structured import build_grammar
        g = build_grammar(params, self.tokenizer, eos, self.config.speculative)
        if copy_given and g is params.grammar:
            import copy
            g = copy.deepcopy(g)
        return g

    def abort_request(self, request_id: str) -> None:
        """Drops a request; for an ``n > 1`` request every sample that is still running."""
        parent = self._parents.pop(request_id, None)
        ids = [request_id] if parent is None else \
            ["%s#%d" % (request_id, i) for i in range(parent["n"])]
        for rid in ids:
            if self.scheduler.abort(rid) is not None and self.runner.suffix_cache is not None:
                self.runner.suffix_cache.stop_request(rid)
        if self.runner.suffix_cache is not None:
            self.runner.suffix_cache.stop_request(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_work() or self._pending is not None

    # ------------------------------------------------------------------- step
    def step(self, partial: bool = False) -> list[RequestOutput]:
        """One scheduling + model step. Returns the requests that finished; with
        ``partial`` also an unfinished ``RequestOutput`` (cumulative text and tokens) for every
        request that produced tokens in this step, for streaming front ends.

        With ``async_scheduling`` a step is left running on the device and its tokens are
        read by the *next* call, after that call has already scheduled and queued the
        following step (the host's scheduling and batching work then overlaps the GPU)."""
        if self.sleeping_level:
            raise RuntimeError("engine is sleeping; call wake_up() first")
        prev, self._pending = self._pending, None
        st, clock = self.stats, time.perf_counter
        if prev is None:
            t0 = clock()
            out = self.scheduler.schedule()
            t1 = clock()
            st["t_schedule"] += t1 - t0
            if out.is_empty:
                return []
            pend = self.runner.launch(out)
            st["t_launch"] += clock() - t1
            if self._can_run_ahead(out):
                self._pending = pend
                return []
            return self._complete(pend, partial)
        nxt = None
        if self._can_run_ahead(prev.out):
            t0 = clock()
            self.scheduler.advance_provisionally(prev.out)
            out = self.scheduler.schedule()
            t1 = clock()
            st["t_schedule"] += t1 - t0
            if not out.is_empty:
                nxt = self.runner.launch(out, prev)
                st["run_ahead_steps"] += 1
                st["t_launch"] += clock() - t1
        outputs = self._complete(prev, partial)
        self._pending = nxt
        return outputs

    def _can_run_ahead(self, out) -> bool:
        """A step may be left in flight when the next step can be scheduled without knowing
        its tokens: no drafting (the accepted length decides the next position) and device
        sampling for every request that samples. Prompt chunks, requests that finish their
        prompt in this step and newly admitted requests are all fine."""
        if not self.config.scheduler.async_scheduling or self.config.speculative is not None:
            return False
        for s in out.scheduled:
            sp = s.request.sampling_params
            if s.samples and (s.num_draft or sp.needs_full_logits or sp.stop):
                return False        # (a stop string is looked for in the text, on the host)
            if sp.prompt_logprobs is not None and s.start < s.request.num_prompt_tokens:
                return False        # its prompt rows are read back when the step completes
        return True

    def _complete(self, pend, partial: bool) -> list[RequestOutput]:
        out = pend.out
        t0 = time.perf_counter()
        result = self.runner.finish(pend)
        t1 = time.perf_counter()
        before = None
        if result.logprobs:
            before = {s.request.request_id: len(s.request.output_token_ids)
                      for s in out.scheduled if s.request.request_id in result.logprobs}
        finished = self.scheduler.update_from_output(out, result.new_tokens, result.drafts)
        if before:
            for s in out.scheduled:
                req = s.request
                if req.request_id not in before:
                    continue
                n = len(req.output_token_ids) - before[req.request_id]   # a stop may cut the step short
                lps, tops = result.logprobs[req.request_id]
                if req.output_logprobs is None:
                    req.output_logprobs, req.output_top_logprobs = [], []
                req.output_logprobs.extend(lps[:n])
                req.output_top_logprobs.extend(tops[:n])
        self.stats["t_wait"] += t1 - t0
        self.stats["t_update"] += time.perf_counter() - t1
        self.step_count += 1
        self.stats["steps"] += 1
        for s in out.scheduled:
            if s.start < s.request.num_prompt_tokens:
                self.stats["prompt_tokens"] += min(s.num_tokens,
                                                   s.request.num_prompt_tokens - s.start)
            if s.num_draft:
                self.stats["draft_tokens"] += s.num_draft
                acc = len(result.new_tokens.get(s.request.request_id, [None])) - 1
                for name, n in (("drafted_per_position", s.num_draft),
                                ("accepted_per_position", acc)):
                    hist = self.stats[name]
                    if len(hist) < n:
                        hist.extend([0] * (n - len(hist)))
                    for i in range(n):
                        hist[i] += 1
        self.stats["sp_steps" if result.mode == "sp" else "tp_steps"] += 1
        for toks in result.new_tokens.values():
            self.stats["generation_tokens"] += len(toks)
            self.stats["accepted_tokens"] += len(toks) - 1
        outputs = []
        if partial:
            done_ids = {r.request_id for r in finished}
            for s in out.scheduled:
                req = s.request
                if req.request_id in done_ids or not result.new_tokens.get(req.request_id) or \
                        req.status.finished:
                    continue
                outputs.append(RequestOutput(req.parent_id or req.request_id, req.prompt,
                                             req.prompt_token_ids, [self._completion(req)], False,
                                             req.metrics, num_cached_tokens=req.num_cached_tokens))
        for req in finished:
            if self.runner.suffix_cache is not None:
                self.runner.suffix_cache.stop_request(req.request_id)
            ro = self._finalize(req)
            if ro is not None:
                outputs.append(ro)
        return outputs

    def get_stats(self) -> dict:
        """Load figures a router needs: queue lengths and KV-cache utilisation."""
        d = dict(self.stats)
        if self.device.type == "cuda":
            from ..ops import native
            d["comm_timeouts"] = native.timeout_count()
        d.update(running=len(self.scheduler.running), waiting=len(self.scheduler.waiting),
                 kv_cache_usage=float(self.kv_manager.usage), num_blocks=self.num_blocks,
                 sleeping_level=self.sleeping_level)
        return d

    def _completion(self, req: Request) -> CompletionOutput:
        text = req.stop_text if req.stop_text is not None else self.tokenizer.decode(
            req.output_token_ids, skip_special_tokens=req.sampling_params.skip_special_tokens)
        lps = req.output_logprobs
        return CompletionOutput(req.sample_index, text, list(req.output_token_ids),
                                req.finish_reason, list(lps) if lps is not None else None,
                                sum(lps) if lps else None,
                                list(req.output_top_logprobs) if lps is not None else None)

    def _finalize(self, req: Request) -> Optional[RequestOutput]:
        comp = self._completion(req)
        if req.parent_id is None:
            return RequestOutput(req.request_id, req.prompt, req.prompt_token_ids, [comp], True,
                                 req.metrics, prompt_logprobs=req.prompt_logprobs,
                                 num_cached_tokens=req.num_cached_tokens)
        parent = self._parents[req.parent_id]
        parent["done"][req.sample_index] = (comp, req.metrics)
        if len(parent["done"]) < parent["n"]:
            return None
        del self._parents[req.parent_id]
        comps = [parent["done"][i][0] for i in range(parent["n"])]
        return RequestOutput(req.parent_id, parent["prompt"], parent["ids"], comps, True,
                             parent["done"][0][1], num_cached_tokens=req.num_cached_tokens)

    # ------------------------------------------------------------ sleep / wake
    def sleep(self, level: int = 1) -> None:
        """Level 1 frees the KV cache; level 2 also moves the weights (and the drafter's)
        to host memory (reference: arctic_inference/server/worker.py:275-390,
        arctic_inference/vllm/patches.py:284-310)."""
        if self.scheduler.has_work() or self._pending is not None:
            raise RuntimeError("cannot sleep with unfinished requests")
        from .sleep import sleep_engine
        sleep_engine(self, level)

    def wake_up(self, tags: Optional[Iterable[str]] = None) -> None:
        from .sleep import wake_engine
        wake_engine(self, tags)

    def reset_prefix_cache(self) -> None:
        self.kv_manager.reset_prefix_cache()
