"""Sampling from truncated distributions (top-k / top-p / grammar masks) and log-probabilities.

No case materialises a probability vector or sorts a row: greedy and plain temperature
sampling run the fused arg-max / Gumbel-max kernel on the raw logits; requests that truncate
the distribution first pass through the selection kernel (``ops.topk_topp_mask``: the k-th
largest logit and the top-p cut are found by counting and summing passes over the row, which
stays in L2), then through the same Gumbel-max kernel. ``apply_top_k_top_p`` is the sort-based
formulation of the same truncation, kept as the oracle of the tests."""

from __future__ import annotations

import zlib

import numpy as np
import torch


def apply_top_k_top_p(logits: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor):
    """logits [B, V] fp32; top_k int64 [B] (<=0: off); top_p fp32 [B]."""
    V = logits.shape[-1]
    sorted_logits, order = logits.sort(dim=-1, descending=True)
    k = torch.where(top_k > 0, top_k, torch.full_like(top_k, V)).clamp(max=V)
    ranks = torch.arange(V, device=logits.device).unsqueeze(0)
    mask = ranks >= k.unsqueeze(1)
    probs = sorted_logits.masked_fill(mask, float("-inf")).softmax(-1)
    cum = probs.cumsum(-1)
    mask |= (cum - probs) > top_p.unsqueeze(1)
    sorted_logits = sorted_logits.masked_fill(mask, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)


def apply_grammar_masks(lf: torch.Tensor, sched, rows) -> torch.Tensor:
    """Set the logits of tokens a request's grammar forbids to -inf. With a draft under
    verification, row j of the request is masked for the state after draft[:j]."""
    out = lf
    for s, rr in zip(sched, rows):
        g = getattr(s.request, "grammar", None)
        if g is None or not rr:
            continue
        draft = s.request.spec_token_ids[:s.num_draft] if s.num_draft else []
        for row, allowed in zip(rr, g.allowed_along(draft)):
            if allowed is None:
                continue
            if out is lf:
                out = lf.clone()
            keep = np.asarray(allowed, dtype=np.int64)
            keep = torch.from_numpy(keep[(keep >= 0) & (keep < lf.shape[-1])]).to(lf.device)
            masked = torch.full_like(out[row], float("-inf"))
            if keep.numel():
                masked[keep] = out[row, keep]
            out[row] = masked
    return out


def apply_penalties(lf: torch.Tensor, sched, rows) -> torch.Tensor:
    """Repetition / presence / frequency penalties and logit bias on the raw logits (before
    temperature), for the requests that ask for them. Row j of a request under verification
    counts the draft tokens before it as generated."""
    out = lf
    V = lf.shape[-1]
    for s, rr in zip(sched, rows):
        sp = s.request.sampling_params
        if not rr or not (sp.presence_penalty or sp.frequency_penalty or
                          sp.repetition_penalty != 1.0 or sp.logit_bias):
            continue
        if out is lf:
            out = lf.clone()
        req = s.request
        draft = list(req.spec_token_ids[:s.num_draft]) if s.num_draft else []
        for j, row in enumerate(rr):
            generated = [t for t in list(req.output_token_ids) + draft[:j] if 0 <= t < V]
            x = out[row]
            if sp.repetition_penalty != 1.0:
                seen = sorted({t for t in req.prompt_token_ids if 0 <= t < V} | set(generated))
                if seen:
                    idx = torch.tensor(seen, dtype=torch.int64, device=x.device)
                    v = x[idx]
                    x[idx] = torch.where(v > 0, v / sp.repetition_penalty, v * sp.repetition_penalty)
            if generated and (sp.presence_penalty or sp.frequency_penalty):
                ids, counts = np.unique(np.asarray(generated, dtype=np.int64), return_counts=True)
                idx = torch.from_numpy(ids).to(x.device)
                cnt = torch.from_numpy(counts.astype(np.float32)).to(x.device)
                x[idx] -= sp.frequency_penalty * cnt + sp.presence_penalty
            if sp.logit_bias:
                keep = [(t, b) for t, b in sp.logit_bias.items() if 0 <= t < V]
                if keep:
                    idx = torch.tensor([t for t, _ in keep], dtype=torch.int64, device=x.device)
                    x[idx] += torch.tensor([b for _, b in keep], dtype=x.dtype, device=x.device)
    return out


def row_seed(request, j: int) -> int:
    """Noise key of the j-th row a request samples in this step: its own seed (or a hash of its
    id) and its token index, so a draw depends neither on the step's other requests nor on the
    previous draws of the same request."""
    sp = request.sampling_params
    base = sp.seed if sp.seed is not None else zlib.crc32(request.request_id.encode()) & 0xFFFFFFF
    return (base * 1000003 + request.num_tokens + j) & 0x7FFFFFFFFFFFFFFF


def sample_full(logits: torch.Tensor, sched, rows) -> torch.Tensor:
    """Sampling from distributions truncated by top-k / top-p / grammar masks. The selection
    kernel leaves the temperature-scaled logits of the kept tokens and -inf elsewhere; they go
    through the same per-row Gumbel-max kernel as plain sampling (a masked token's -inf never
    wins), keyed per row by :func:`row_seed`."""
    from .. import ops
    B = logits.shape[0]
    dev = logits.device
    lf = apply_penalties(logits.float(), sched, rows)
    lf = apply_grammar_masks(lf, sched, rows)
    temp = np.ones(B, dtype=np.float32)
    min_p = np.zeros(B, dtype=np.float32)
    top_k = np.zeros(B, dtype=np.int64)
    top_p = np.ones(B, dtype=np.float32)
    draw = np.zeros(B, dtype=np.float32)      # 1: sample, 0: arg-max
    seeds = np.zeros(B, dtype=np.int64)
    for s, rr in zip(sched, rows):
        sp = s.request.sampling_params
        for j, row in enumerate(rr):
            temp[row] = max(sp.temperature, 1e-5)
            top_k[row] = sp.top_k
            top_p[row] = sp.top_p
            min_p[row] = sp.min_p
            draw[row] = 0.0 if sp.greedy else 1.0
            seeds[row] = row_seed(s.request, j)
    lf = ops.topk_topp_mask(lf.contiguous(), torch.from_numpy(temp).to(dev),
                            torch.from_numpy(top_k).to(dev), torch.from_numpy(top_p).to(dev))
    if min_p.any():
        # a token stays iff its probability is at least min_p times the most likely one's:
        # in (scaled) logit space, within ln(min_p) of the row's maximum
        floor = lf.max(-1, keepdim=True).values + \
            torch.log(torch.from_numpy(min_p).to(dev).clamp(min=1e-30)).unsqueeze(1)
        lf = lf.masked_fill(lf < floor, float("-inf"))
    ids, _ = ops.argmax_sample(lf, torch.from_numpy(draw).to(dev), torch.from_numpy(seeds).to(dev))
    return ids


def compute_logprobs(logits: torch.Tensor, token_ids: torch.Tensor, k: int):
    """Log-probabilities of chosen tokens and of the top-k alternatives."""
    lp = logits.float().log_softmax(-1)
    chosen = lp.gather(-1, token_ids.unsqueeze(-1)).squeeze(-1)
    topv, topi = lp.topk(max(k, 1), dim=-1)
    return chosen, topv, topi
