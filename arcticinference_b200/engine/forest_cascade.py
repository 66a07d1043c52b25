"""Forest cascade attention: decode batches whose requests share KV-cache prefixes (same
system prompt, parallel samples of one prompt, tree search) read each shared prefix once
per group instead of once per request.

The reference implements this as a replacement attention backend: permute queries so group
members are adjacent, run one FlashAttention call over group prefixes, one over per-request
suffixes, and merge the two by log-sum-exp
(arctic_inference/vllm/attention/flash_attn_forest_cascade.py:1303-1478 grouping,
:1677-1807 forward). Here it is host-side planning only: the attention kernel already
executes an arbitrary list of (query rows, key range, block-table row) work items and folds
partial results that target the same token, so a cascade is just a different work list --

* requests are ordered so that members of a group are adjacent in the batch;
* one work item per group covers all member query rows against the group's prefix blocks
  (every prefix key precedes every member query, so no mask applies): partial 0;
* one work item per member covers its own rows against its remaining blocks, causal: partial 1;
* the existing merge kernel combines the two partials per token.

Grouping: requests are sorted by their block-id rows (only blocks completely filled by
context count), the common prefix of adjacent rows is measured in blocks, and a range of
the sorted order is split recursively at its weakest link when that increases the number of
(request x shared block) reads saved.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from ..config import ForestCascadeConfig

TILE_KEYS = 128


@dataclass
class CascadeGroup:
    members: list            # indices into the batch (in sorted order)
    prefix_blocks: int       # shared blocks


@dataclass
class CascadePlan:
    order: list                       # new batch order (indices into the original batch)
    groups: list = field(default_factory=list)   # CascadeGroup over positions in `order`
    saved_block_reads: int = 0

    @property
    def non_singleton(self) -> list:
        return [g for g in self.groups if len(g.members) > 1 and g.prefix_blocks > 0]


def _lcp(a: Sequence[int], b: Sequence[int], limit: int) -> int:
    n = 0
    m = min(len(a), len(b), limit)
    while n < m and a[n] == b[n]:
        n += 1
    return n


def plan_groups(block_tables: Sequence[Sequence[int]], context_lens: Sequence[int],
                block_size: int, cfg: ForestCascadeConfig) -> Optional[CascadePlan]:
    """Group the requests of a batch by shared prefix. ``context_lens[i]`` is the number of
    cached tokens *before* request i's query tokens; only blocks that these fill completely
    can be shared. Returns None when the gates say a cascade is not worth it."""
    R = len(block_tables)
    if R < max(cfg.min_batch_size, 2):
        return None
    full = [int(c) // block_size for c in context_lens]
    rows = [tuple(block_tables[i][:full[i]]) for i in range(R)]
    order = sorted(range(R), key=lambda i: rows[i])
    lcp = [0] * R  # lcp[k] = shared blocks between order[k-1] and order[k]
    for k in range(1, R):
        a, b = order[k - 1], order[k]
        lcp[k] = _lcp(rows[a], rows[b], min(full[a], full[b]))

    groups: list[CascadeGroup] = []

    def range_prefix(lo: int, hi: int) -> int:
        # shared blocks of order[lo:hi]
        if hi - lo == 1:
            return 0
        return min(lcp[lo + 1:hi])

    def value(lo: int, hi: int) -> int:
        # block reads saved by treating order[lo:hi] as one group
        size = hi - lo
        return size * range_prefix(lo, hi) if size >= cfg.min_group_size else 0

    def emit(lo: int, hi: int) -> None:
        size = hi - lo
        if size >= 2:
            inner = lcp[lo + 1:hi]
            cut = lo + 1 + int(np.argmin(inner))        # weakest link: split between cut-1, cut
            if value(lo, cut) + value(cut, hi) > value(lo, hi) or \
                    (value(lo, hi) == 0 and size > 2):
                emit(lo, cut)
                emit(cut, hi)
                return
        pre = range_prefix(lo, hi) if size >= cfg.min_group_size else 0
        groups.append(CascadeGroup(list(range(lo, hi)), pre))

    emit(0, R)
    plan = CascadePlan(order=order, groups=groups)
    ns = plan.non_singleton
    if not ns:
        return None
    if len(ns) > cfg.max_non_singleton_groups:
        return None
    covered = sum(len(g.members) for g in ns)
    if covered < cfg.min_non_singleton_fraction * R:
        return None
    if not any(g.prefix_blocks >= cfg.min_additional_prefix_blocks for g in ns):
        return None
    plan.saved_block_reads = sum((len(g.members) - 1) * g.prefix_blocks for g in ns)
    return plan


def build_cascade_work(plan: CascadePlan, q_lens: Sequence[int], kv_lens: Sequence[int],
                       block_tables: Sequence[Sequence[int]], block_size: int, G: int):
    """Work list and block table for a planned batch. ``q_lens / kv_lens / block_tables`` are in
    the *new* batch order (``plan.order`` applied). Returns
    (work [n,8] int32, tok_splits [T] int32, table [rows, width] int32, max_splits)."""
    tpt = 128 // G
    R = len(q_lens)
    starts = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int64)
    T = int(starts[-1])
    tok_splits = np.ones(max(T, 1), dtype=np.int32)
    rows = []
    table_rows = []          # block-table rows: first one per request suffix, then group prefixes
    width = max(len(b) for b in block_tables)
    # per-request rows (suffix tables are the request's own table shifted by the prefix)
    prefix_of = [0] * R
    for g in plan.groups:
        if len(g.members) > 1 and g.prefix_blocks > 0:
            for m in g.members:
                prefix_of[m] = g.prefix_blocks
    for i in range(R):
        t = list(block_tables[i][prefix_of[i]:])
        table_rows.append(t)
    for i in range(R):
        pre_tok = prefix_of[i] * block_size
        kl = kv_lens[i] - pre_tok
        ql = q_lens[i]
        ns = 2 if prefix_of[i] else 1
        for a in range(0, ql, tpt):
            n = min(tpt, ql - a)
            rows.append((i, int(starts[i]) + a, n, kl - ql + a, 0, kl, ns - 1, ns))
        if ns == 2:
            tok_splits[starts[i]:starts[i + 1]] = 2
    for g in plan.groups:
        if len(g.members) <= 1 or g.prefix_blocks <= 0:
            continue
        row = len(table_rows)
        table_rows.append(list(block_tables[g.members[0]][:g.prefix_blocks]))
        pre_tok = g.prefix_blocks * block_size
        t0, t1 = int(starts[g.members[0]]), int(starts[g.members[-1] + 1])
        for a in range(t0, t1, tpt):
            n = min(tpt, t1 - a)
            # q position = prefix length: every prefix key is visible to every member row
            rows.append((row, a, n, pre_tok, 0, pre_tok, 0, 2))
    width = max(width, max(len(r) for r in table_rows))
    table = np.zeros((len(table_rows), width), dtype=np.int32)
    for i, r in enumerate(table_rows):
        table[i, :len(r)] = r
    work = np.asarray(rows, dtype=np.int32).reshape(-1, 8)
    return work, tok_splits, table, 2


def gate(cfg: ForestCascadeConfig, q_lens: Sequence[int], all_sampling: bool) -> bool:
    """Cheap checks before any grouping work: decode-shaped, enough requests."""
    return (cfg.enabled and all_sampling and len(q_lens) >= cfg.min_batch_size and
            max(q_lens) <= cfg.max_query_len)
