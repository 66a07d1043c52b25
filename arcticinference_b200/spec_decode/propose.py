"""Drafting for the next step: Arctic speculator on the GPU, suffix trees on the host, or both.

After a step has sampled, every request that produced a token gets a draft:

* ``arctic`` / ``mlp_speculator``: the draft model runs once for all such requests, seeded with
  the target's hidden state at each request's last accepted position and the token just sampled
  (arctic_inference/vllm/spec_dec/arctic_proposer.py:130-209);
* ``suffix``: the request's local tree and the global tree are queried with the last
  ``suffix_cache_max_depth`` tokens (arctic_inference/vllm/model_runner.py:1128-1188);
* hybrid (``arctic`` + ``enable_suffix_decoding``): the suffix draft wins when its score reaches
  the speculator's draft length, otherwise the speculator's draft is used
  (model_runner.py:1008-1023).

Which requests may carry a draft into the next step is decided by the scheduler through
``SpeculativeConfig.effective_draft_limit``. Every rank of a multi-GPU engine runs this code
on identical inputs and therefore produces identical drafts.
"""

from __future__ import annotations

import logging

import torch

from .. import ops

logger = logging.getLogger(__name__)


def attach_speculation(engine) -> None:
    cfg = engine.config.speculative
    runner = engine.runner
    if cfg.uses_arctic:
        from ..models.speculator import SpeculatorConfig, build_speculator
        m = engine.config.model
        if cfg.model in (None, "random", "dummy") or not __import__("os").path.isdir(str(cfg.model)):
            scfg = SpeculatorConfig(
                n_predict=cfg.num_speculative_tokens or 3, vocab_size=m.vocab_size,
                emb_dim=m.hidden_size, inner_dim=m.hidden_size, proj_dim=m.hidden_size,
                input_hidden_dim=m.hidden_size,
                method="mlp" if cfg.method == "mlp_speculator" else "sum_lstm",
                tie_weights=True, scale_input=True)
            runner.proposer = build_speculator(scfg, runner.device, seed=engine.config.seed + 1)
        else:
            runner.proposer = build_speculator(cfg.model, runner.device)
        comm = getattr(engine, "comm", None)
        if comm is not None and comm.ways > 1 and runner.proposer.shard_heads(comm):
            logger.info("speculator: LM heads sharded by vocabulary over %d ranks", comm.ways)
        if cfg.quantization == "fp8":
            n = runner.proposer.quantize_fp8()
            logger.info("speculator: %d matrices stored as fp8 with per-row scales", n)
        elif runner.device.type == "cuda":
            n = runner.proposer.make_qheads()
            logger.info("speculator: %d fp8 LM-head copies for small batches", n)
        if cfg.num_speculative_tokens is None:
            cfg.num_speculative_tokens = runner.proposer.n_predict
        if runner.proposer.cfg.vocab_size != m.vocab_size:
            logger.warning("speculator vocabulary (%d) differs from the target's (%d)",
                           runner.proposer.cfg.vocab_size, m.vocab_size)
    if cfg.uses_suffix:
        from ..suffix_decoding import SuffixDecodingCache
        runner.suffix_cache = SuffixDecodingCache(cfg.suffix_cache_max_depth,
                                                  cfg.suffix_cache_max_requests)
    runner.spec_stats = {"arctic_drafts": 0, "suffix_drafts": 0, "draft_tokens": 0}


def _suffix_draft(runner, req, cfg):
    cache = runner.suffix_cache
    rid = req.request_id
    if rid not in cache.active_requests:
        cache.start_request(rid, req.prompt_token_ids)
        req._suffix_seen = 0
    seen = getattr(req, "_suffix_seen", 0)
    out = req.output_token_ids
    if len(out) > seen:
        cache.add_active_response(rid, out[seen:])
        req._suffix_seen = len(out)
    depth = cfg.suffix_cache_max_depth
    toks = req.all_token_ids
    pattern = toks[-depth:]
    max_model_len = runner.config.scheduler.max_model_len
    limit = cfg.suffix_speculative_tokens or cfg.num_speculative_tokens or depth
    max_spec = min(limit, max_model_len - len(toks) - 1)
    if max_spec <= 0:
        return None
    return cache.speculate(rid, pattern, max_spec_tokens=max_spec,
                           max_spec_factor=cfg.suffix_max_spec_factor,
                           max_spec_offset=cfg.suffix_max_spec_offset,
                           min_token_prob=cfg.suffix_min_token_prob)


def propose_drafts(runner, sched, rows, new_tokens: dict, hidden: torch.Tensor,
                   accepted_rows: list, arctic: list = None) -> dict:
    """Drafts for the next step. The speculator's heads are queued on the GPU first and their
    tokens start their way to pinned host memory; the suffix trees are then searched on the
    CPU while the GPU drafts, and only after that does the host wait for the speculator's
    tokens (the reference overlaps the same two with a copy stream:
    arctic_inference/vllm/model_runner.py:1323-1628, its mode "B"). Per request the suffix
    draft wins when its score reaches the speculator's draft length, else the speculator's
    draft is used (model_runner.py:1008-1023). ``arctic`` carries the speculator's drafts when
    the step already produced them on the device behind its verification kernel."""
    cfg = runner.config.speculative
    reqs = [s.request for s in sched if s.samples]
    drafts: dict = {}
    if not reqs:
        return drafts
    arctic_dev = arctic_host = arctic_event = None
    if runner.proposer is not None and arctic is None:
        n_predict = cfg.num_speculative_tokens or runner.proposer.n_predict
        idx = torch.tensor(accepted_rows, dtype=torch.int64, device=hidden.device)
        tok = torch.tensor([new_tokens[r.request_id][-1] for r in reqs], dtype=torch.int64,
                           device=hidden.device)
        h = ops.gather_rows(hidden, idx) if hidden.is_cuda else hidden[idx]
        arctic_dev = runner.proposer.propose(h, tok, n_predict)
        if arctic_dev.is_cuda:
            arctic_host = torch.empty(arctic_dev.shape, dtype=arctic_dev.dtype, pin_memory=True)
            arctic_host.copy_(arctic_dev, non_blocking=True)
            arctic_event = torch.cuda.Event()
            arctic_event.record()
        runner.d2h_total += len(reqs) * n_predict * 8

    # suffix search on the CPU (while the GPU drafts)
    suffix: list = [None] * len(reqs)
    if runner.suffix_cache is not None:
        for i, req in enumerate(reqs):
            if req.status.finished:
                continue
            # tokens of this step are not in req.output_token_ids yet: look one step ahead
            saved = req.output_token_ids
            req.output_token_ids = saved + new_tokens[req.request_id]
            try:
                suffix[i] = _suffix_draft(runner, req, cfg)
            finally:
                req.output_token_ids = saved

    if arctic_dev is not None:
        if arctic_event is not None:
            arctic_event.synchronize()
            arctic = arctic_host.tolist()
        else:
            arctic = arctic_dev.tolist()

    threshold = (cfg.num_speculative_tokens or 0) if arctic is not None else 0
    for i, req in enumerate(reqs):
        if req.status.finished:
            continue
        d = None
        sd = suffix[i]
        if sd is not None and sd.token_ids and sd.score >= threshold:
            d = [int(t) for t in sd.token_ids]
            runner.spec_stats["suffix_drafts"] += 1
        if d is None and arctic is not None:
            d = arctic[i]
            runner.spec_stats["arctic_drafts"] += 1
        if d:
            drafts[req.request_id] = d
            runner.spec_stats["draft_tokens"] += len(d)
    return drafts
