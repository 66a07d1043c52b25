"""Python front of the suffix trees.

One *global* tree holds the responses of past requests (FIFO-evicted beyond
``max_cached_requests``); every active request additionally has a *local* tree over
its own prompt + response, which catches self-repetition and copying from the prompt.
``speculate`` asks both and returns the draft with the higher score.

Behavioural parity with arctic_inference/suffix_decoding/cache.py:120-357 (same method
names and arguments); the ``max_depth`` attribute the reference forgets to define
(cache.py:285) exists here.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np


def _load_ext():
    try:
        from . import _C  # noqa: F401
    except ImportError:
        from .. import build
        build.build_suffix_tree()
        from . import _C  # noqa: F401
    return _C


_C = _load_ext()
SuffixTree = _C.SuffixTree


@dataclass
class SuffixDecodingDraft:
    token_ids: list = field(default_factory=list)
    parents: list = field(default_factory=list)
    probs: list = field(default_factory=list)
    score: float = 0.0
    match_len: int = 0

    @classmethod
    def from_native(cls, d) -> "SuffixDecodingDraft":
        return cls(list(d.token_ids), list(d.parents), list(d.probs), float(d.score),
                   int(d.match_len))


def _as_i32(tokens) -> np.ndarray:
    if isinstance(tokens, np.ndarray):
        return np.ascontiguousarray(tokens, dtype=np.int32)
    return np.asarray(tokens, dtype=np.int32)


class SuffixDecodingCache:
    def __init__(self, max_tree_depth: int = 64, max_cached_requests: int = -1):
        if max_cached_requests > 0x7FFFFFFF:
            raise ValueError("max_cached_requests must fit in int32")
        self.max_tree_depth = max_tree_depth
        self.max_depth = max_tree_depth
        self.max_cached_requests = max_cached_requests
        self._global = SuffixTree(max_tree_depth)
        self._local: dict[Hashable, SuffixTree] = {}
        # request id <-> int32 sequence id of its response in the global tree
        self._req_to_seq: "OrderedDict[Hashable, int]" = OrderedDict()
        self._seq_to_req: dict[int, Hashable] = {}
        self._next_seq = 0
        self._prompt_len: dict[Hashable, int] = {}

    # ------------------------------------------------------------------ properties
    @property
    def active_requests(self):
        return self._local.keys()

    @property
    def cached_requests(self):
        return self._req_to_seq.keys()

    @property
    def num_cached_requests(self) -> int:
        return len(self._req_to_seq)

    def global_tree(self) -> SuffixTree:
        return self._global

    # ------------------------------------------------------------------ sequence ids
    def _new_seq_id(self) -> int:
        # int32 ids, wrapping around and skipping ids that are still in use
        while True:
            sid = self._next_seq
            self._next_seq = (self._next_seq + 1) & 0x7FFFFFFF
            if sid not in self._seq_to_req:
                return sid

    def _evict_if_needed(self) -> None:
        if self.max_cached_requests < 0:
            return
        while len(self._req_to_seq) > self.max_cached_requests:
            # oldest cached response that does not belong to a running request
            victim = None
            for rid in self._req_to_seq:
                if rid not in self._local:
                    victim = rid
                    break
            if victim is None:
                return
            self.evict_cached_response(victim)

    # ------------------------------------------------------------------ request lifecycle
    def start_request(self, req_id: Hashable, prompt_token_ids: Sequence[int]) -> None:
        """Begin tracking a request: builds its local tree from the prompt and reserves a
        slot for its response in the global tree."""
        if req_id in self._local:
            raise ValueError("request %r is already active" % (req_id,))
        tree = SuffixTree(self.max_tree_depth)
        prompt = _as_i32(prompt_token_ids)
        tree.extend_ndarray(0, prompt)
        self._local[req_id] = tree
        self._prompt_len[req_id] = int(prompt.size)
        if self.max_cached_requests != 0:
            if req_id in self._req_to_seq:
                self.evict_cached_response(req_id)
            sid = self._new_seq_id()
            self._req_to_seq[req_id] = sid
            self._seq_to_req[sid] = req_id
            self._evict_if_needed()

    def stop_request(self, req_id: Hashable) -> None:
        """Stop tracking a request; its response stays in the global tree until evicted."""
        self._local.pop(req_id, None)
        self._prompt_len.pop(req_id, None)
        self._evict_if_needed()

    def add_active_response(self, req_id: Hashable, token_ids: Sequence[int]) -> None:
        """Append newly generated tokens of an active request to both trees."""
        tree = self._local.get(req_id)
        if tree is None:
            raise ValueError("request %r is not active" % (req_id,))
        toks = _as_i32(token_ids)
        if toks.size == 0:
            return
        tree.extend_ndarray(0, toks)
        sid = self._req_to_seq.get(req_id)
        if sid is not None:
            self._global.extend_ndarray(sid, toks)

    def evict_cached_response(self, req_id: Hashable) -> None:
        sid = self._req_to_seq.pop(req_id, None)
        if sid is None:
            return
        del self._seq_to_req[sid]
        self._global.remove(sid)

    # ------------------------------------------------------------------ speculation
    def speculate(self, req_id: Hashable, context: Sequence[int], max_spec_tokens: Optional[int] = None,
                  max_spec_factor: float = 1.0, max_spec_offset: float = 0.0,
                  min_token_prob: float = 0.1, use_tree_spec: bool = False,
                  use_cached_prompt: bool = True) -> SuffixDecodingDraft:
        """Draft a continuation of ``context`` (the most recent tokens of the request).
        Returns the higher-scoring draft of the request's own tree and the global tree."""
        tree = self._local.get(req_id)
        if tree is None:
            raise ValueError("request %r is not active" % (req_id,))
        if max_spec_tokens is None:
            max_spec_tokens = self.max_depth
        ctx = _as_i32(context)
        if ctx.size > self.max_tree_depth:
            ctx = ctx[-self.max_tree_depth:]
        best = None
        if use_cached_prompt:
            best = tree.speculate_ndarray(ctx, max_spec_tokens, max_spec_factor, max_spec_offset,
                                          min_token_prob, use_tree_spec)
        g = self._global.speculate_ndarray(ctx, max_spec_tokens, max_spec_factor, max_spec_offset,
                                           min_token_prob, use_tree_spec)
        if best is None or g.score > best.score:
            best = g
        return SuffixDecodingDraft.from_native(best)

    def check_integrity(self) -> str:
        err = self._global.check_integrity()
        if err:
            return "global: " + err
        for rid, t in self._local.items():
            err = t.check_integrity()
            if err:
                return "local %r: %s" % (rid, err)
        return ""

    def estimate_memory(self) -> int:
        return self._global.estimate_memory() + sum(t.estimate_memory() for t in self._local.values())
