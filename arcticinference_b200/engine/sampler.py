"""Full-distribution sampling (top-k / top-p / log-probabilities).

The common cases (greedy, plain temperature sampling) never materialise a
probability vector: they run the fused arg-max / Gumbel-max kernel on the raw
logits. Requests that truncate the distribution take this slower path, which
is framework-level PyTorch on the gathered logits."""

from __future__ import annotations

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


def sample_full(logits: torch.Tensor, sched, rows) -> torch.Tensor:
    B = logits.shape[0]
    dev = logits.device
    lf = apply_grammar_masks(logits.float(), sched, rows)
    raw = lf
    temp = torch.ones(B, device=dev)
    top_k = torch.zeros(B, dtype=torch.int64, device=dev)
    top_p = torch.ones(B, device=dev)
    greedy = torch.zeros(B, dtype=torch.bool, device=dev)
    seed = 0
    for s, rr in zip(sched, rows):
        sp = s.request.sampling_params
        for row in rr:
            temp[row] = max(sp.temperature, 1e-5)
            top_k[row] = sp.top_k
            top_p[row] = sp.top_p
            greedy[row] = sp.greedy
        if rr and sp.seed is not None:
            seed = seed * 31 + sp.seed + s.request.num_tokens
    lf = apply_top_k_top_p(lf / temp.unsqueeze(1), top_k, top_p)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed & 0x7FFFFFFF)
    probs = lf.softmax(-1)
    sampled = torch.multinomial(probs, 1, generator=gen).squeeze(1)
    return torch.where(greedy, raw.argmax(-1), sampled)


def compute_logprobs(logits: torch.Tensor, token_ids: torch.Tensor, k: int):
    """Log-probabilities of chosen tokens and of the top-k alternatives."""
    lp = logits.float().log_softmax(-1)
    chosen = lp.gather(-1, token_ids.unsqueeze(-1)).squeeze(-1)
    topv, topi = lp.topk(max(k, 1), dim=-1)
    return chosen, topv, topi
