"""Offline simulator of suffix decoding (no GPU, no model).

Replays recorded (prompt, response) token sequences: at every step it drafts from
the suffix trees, verifies the draft against the recorded continuation (the longest
root-to-node path of the draft tree that agrees with the ground truth is accepted,
plus one "bonus" token the target model would have produced anyway), feeds the
accepted tokens back into the trees and measures acceptance and host time.

    python -m arcticinference_b200.suffix_decoding.simulator --synthetic \
        --num-requests 256 --prompt-len 512 --response-len 256 --train-requests 128

Metrics per configuration (as in arctic_inference/suffix_decoding/simulator.py:255-291):
``accept_rate`` (accepted / drafted), ``mean_accepted_len`` (tokens per step incl. bonus),
``req_speedup`` (response length / steps), ``spec_ms_per_tok``, ``update_ms_per_tok``.
"""

from __future__ import annotations

import argparse
import itertools
import json
import time
from dataclasses import dataclass, asdict
from typing import Optional, Sequence

import numpy as np

from .cache import SuffixDecodingCache


# --------------------------------------------------------------------------- data
def synthetic_requests(num_requests: int = 256, prompt_len: int = 512, response_len: int = 256,
                       vocab: int = 128256, zipf_s: float = 1.1, window: int = 32,
                       reuse_prob: float = 0.5, ngram_min: int = 8, ngram_max: int = 24,
                       seed: int = 0):
    """Token streams drawn from Zipf(s) in which every ``window`` tokens, with probability
    ``reuse_prob``, a previously emitted n-gram (8-24 tokens) is copied instead."""
    rng = np.random.default_rng(seed)
    ranks = np.arange(1, vocab + 1, dtype=np.float64)
    pmf = ranks ** (-zipf_s)
    cdf = np.cumsum(pmf / pmf.sum())
    emitted: list[np.ndarray] = []

    def draw(n):
        return np.searchsorted(cdf, rng.random(n)).astype(np.int32).clip(0, vocab - 1)

    def stream(n):
        out = np.empty(0, dtype=np.int32)
        while out.size < n:
            if emitted and rng.random() < reuse_prob:
                src = emitted[rng.integers(len(emitted))]
                k = int(rng.integers(ngram_min, ngram_max + 1))
                if src.size > k:
                    s = int(rng.integers(0, src.size - k))
                    out = np.concatenate([out, src[s:s + k]])
            fresh = draw(window)
            out = np.concatenate([out, fresh])
        out = out[:n]
        emitted.append(out)
        return out

    return [(stream(prompt_len), stream(response_len)) for _ in range(num_requests)]


# --------------------------------------------------------------------------- replay
@dataclass
class SimConfig:
    max_depth: int = 64
    max_spec_tokens: int = 32
    max_spec_factor: float = 1.0
    max_spec_offset: float = 0.0
    min_token_prob: float = 0.1
    use_tree_spec: bool = False
    use_cached_prompt: bool = True
    max_cached_requests: int = -1


@dataclass
class SimResult:
    num_requests: int = 0
    num_steps: int = 0
    num_drafted: int = 0
    num_accepted: int = 0
    num_output_tokens: int = 0
    spec_s: float = 0.0
    update_s: float = 0.0

    def summary(self) -> dict:
        steps = max(self.num_steps, 1)
        toks = max(self.num_output_tokens, 1)
        return {
            "accept_rate": self.num_accepted / max(self.num_drafted, 1),
            "mean_accepted_len": self.num_output_tokens / steps,
            "req_speedup": self.num_output_tokens / steps,
            "spec_ms_per_tok": 1e3 * self.spec_s / toks,
            "update_ms_per_tok": 1e3 * self.update_s / toks,
            "spec_us_per_step": 1e6 * self.spec_s / steps,
            "num_steps": self.num_steps,
            "num_output_tokens": self.num_output_tokens,
        }


def verify_draft(token_ids: Sequence[int], parents: Sequence[int], truth: Sequence[int]) -> int:
    """Length of the longest root-to-node path of the draft tree that equals a prefix of
    ``truth``. Children of draft token p are the tokens whose parent index is p."""
    n = len(token_ids)
    if n == 0:
        return 0
    best = 0
    depth = [0] * n
    ok = [False] * n
    for i in range(n):
        p = parents[i]
        d = 0 if p < 0 else depth[p] + 1
        depth[i] = d
        parent_ok = True if p < 0 else ok[p]
        ok[i] = parent_ok and d < len(truth) and token_ids[i] == truth[d]
        if ok[i]:
            best = max(best, d + 1)
    return best


def simulate_request(cache: SuffixDecodingCache, req_id, prompt: np.ndarray, response: np.ndarray,
                     cfg: SimConfig, res: SimResult) -> list:
    t0 = time.perf_counter()
    cache.start_request(req_id, prompt)
    res.update_s += time.perf_counter() - t0
    history = np.concatenate([prompt, response]).astype(np.int32)
    plen = prompt.size
    pos = 0  # response tokens produced so far
    produced = []
    n = response.size
    # the first response token comes from the prefill step
    t0 = time.perf_counter()
    cache.add_active_response(req_id, response[:1])
    res.update_s += time.perf_counter() - t0
    produced.append(int(response[0]))
    pos = 1
    while pos < n:
        ctx = history[max(0, plen + pos - cfg.max_depth):plen + pos]
        t0 = time.perf_counter()
        d = cache.speculate(req_id, ctx, max_spec_tokens=min(cfg.max_spec_tokens, n - pos - 1),
                            max_spec_factor=cfg.max_spec_factor,
                            max_spec_offset=cfg.max_spec_offset,
                            min_token_prob=cfg.min_token_prob, use_tree_spec=cfg.use_tree_spec,
                            use_cached_prompt=cfg.use_cached_prompt)
        res.spec_s += time.perf_counter() - t0
        truth = response[pos:]
        acc = verify_draft(d.token_ids, d.parents, truth)
        new = response[pos:pos + acc + 1]  # accepted tokens + the bonus token
        t0 = time.perf_counter()
        cache.add_active_response(req_id, new)
        res.update_s += time.perf_counter() - t0
        produced.extend(int(x) for x in new)
        res.num_steps += 1
        res.num_drafted += len(d.token_ids)
        res.num_accepted += acc
        pos += new.size
    res.num_output_tokens += n - 1
    res.num_requests += 1
    t0 = time.perf_counter()
    cache.stop_request(req_id)
    res.update_s += time.perf_counter() - t0
    assert produced == [int(x) for x in response], "replay must reproduce the recorded response"
    return produced


def run(requests, train_requests: int, cfg: SimConfig, check_integrity: bool = False) -> dict:
    cache = SuffixDecodingCache(cfg.max_depth, cfg.max_cached_requests)
    # seed the global tree with the responses of the training split
    for i in range(train_requests):
        p, r = requests[i]
        cache.start_request(("train", i), p[:1])
        cache.add_active_response(("train", i), r)
        cache.stop_request(("train", i))
    res = SimResult()
    for i in range(train_requests, len(requests)):
        p, r = requests[i]
        simulate_request(cache, ("eval", i), p, r, cfg, res)
    if check_integrity:
        err = cache.check_integrity()
        if err:
            raise RuntimeError("suffix tree integrity: " + err)
    out = res.summary()
    out["config"] = asdict(cfg)
    out["memory_bytes"] = cache.estimate_memory()
    return out


def load_jsonl(path: str, tokenizer=None):
    """Rows with ``prompt_token_ids``/``response_token_ids`` (or ``prompt``/``response`` text
    when a tokenizer is given)."""
    reqs = []
    with open(path) as f:
        for line in f:
            row = json.loads(line)
            if "prompt_token_ids" in row:
                p, r = row["prompt_token_ids"], row["response_token_ids"]
            else:
                p, r = tokenizer.encode(row["prompt"]), tokenizer.encode(row["response"])
            reqs.append((np.asarray(p, dtype=np.int32), np.asarray(r, dtype=np.int32)))
    return reqs


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--dataset", type=str, default=None, help="JSONL of token id pairs")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--num-requests", type=int, default=256)
    ap.add_argument("--train-requests", type=int, default=128)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--response-len", type=int, default=256)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max-depth", type=int, nargs="+", default=[64])
    ap.add_argument("--max-spec-tokens", type=int, nargs="+", default=[32])
    ap.add_argument("--max-spec-factor", type=float, nargs="+", default=[1.0])
    ap.add_argument("--max-spec-offset", type=float, nargs="+", default=[0.0])
    ap.add_argument("--min-token-prob", type=float, nargs="+", default=[0.1])
    ap.add_argument("--use-tree-spec", type=int, nargs="+", default=[0])
    ap.add_argument("--check-integrity", action="store_true")
    a = ap.parse_args(argv)
    if a.dataset:
        requests = load_jsonl(a.dataset)
    else:
        requests = synthetic_requests(a.num_requests, a.prompt_len, a.response_len, a.vocab,
                                      seed=a.seed)
    grid = itertools.product(a.max_depth, a.max_spec_tokens, a.max_spec_factor, a.max_spec_offset,
                             a.min_token_prob, a.use_tree_spec)
    for depth, spec, factor, offset, prob, tree in grid:
        cfg = SimConfig(depth, spec, factor, offset, prob, bool(tree))
        print(json.dumps(run(requests, min(a.train_requests, len(requests) - 1), cfg,
                             a.check_integrity)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
