"""Ops of the draft models (Arctic speculators) and of greedy draft verification.
CUDA tensors run the kernels in ``csrc/speculator.cu``; CPU tensors run the PyTorch
restatements below, which are also the test oracles."""

from __future__ import annotations


import torch
import torch.nn.functional as F

from . import launch_counter


def _nat():
    from . import native
    return native


# ------------------------------------------------------------------------- references
def spec_ln_ref(x, w=None, b=None, eps=1e-6, out_scale=1.0):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * out_scale
    if w is not None:
        y = y * w.float()
    if b is not None:
        y = y + b.float()
    return y.to(x.dtype)


def _gelu(x, tanh_approx):
    return F.gelu(x, approximate="tanh" if tanh_approx else "none")


def mlp_spec_step_ref(proj, emb, tok, emb_scale, ln_w, ln_b, eps=1e-6, tanh_approx=False):
    z = proj.float() + emb_scale * emb[tok].float()
    y = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps)
    if ln_w is not None:
        y = y * ln_w.float()
    if ln_b is not None:
        y = y + ln_b.float()
    return _gelu(y, tanh_approx).to(proj.dtype)


def sum_lstm_ref(gates, emb, tok, alpha, prev_c, w_cell, b_cell, w_state, b_state, eps=1e-6,
                 tanh_approx=False):
    D = gates.shape[-1] // 4
    e = emb[tok].float()
    if e.shape[-1] == D:
        e = e.repeat(1, 4)
    g = gates.float() + alpha * e
    f, i, o, c = g[:, :D], g[:, D:2 * D], g[:, 2 * D:3 * D], g[:, 3 * D:]

    def ln(x, w, b):
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            y = y * w.float()
        if b is not None:
            y = y + b.float()
        return y

    cp = prev_c.float() if prev_c is not None else torch.zeros_like(f)
    c_new = cp * torch.sigmoid(f) + _gelu(ln(c, w_cell, b_cell), tanh_approx) * torch.sigmoid(i)
    c_new = c_new.to(gates.dtype)
    h = _gelu(ln(c_new.float(), w_state, b_state), tanh_approx) * torch.sigmoid(o)
    return c_new, h.to(gates.dtype)


def verify_greedy_ref(input_ids, target, row_start, num_draft, max_draft):
    R = len(row_start)
    accepted = torch.zeros(R, dtype=torch.int32)
    next_tok = torch.zeros(R, dtype=torch.int64)
    sel_row = torch.zeros(R, dtype=torch.int64)
    out = torch.full((R, max_draft + 1), -1, dtype=torch.int64)
    ids, tgt = input_ids.tolist(), target.tolist()
    for r in range(R):
        s, nd = int(row_start[r]), int(num_draft[r])
        if s < 0:
            continue
        a = 0
        while a < nd and ids[s + a + 1] == tgt[s + a]:
            a += 1
        accepted[r] = a
        next_tok[r] = tgt[s + a]
        sel_row[r] = s + a
        out[r, :a + 1] = torch.tensor(tgt[s:s + a + 1])
    dev = input_ids.device
    return accepted.to(dev), next_tok.to(dev), sel_row.to(dev), out.to(dev)


# ----------------------------------------------------------------------------- wrappers
def spec_ln(x, w=None, b=None, eps=1e-6, out_scale=1.0):
    if not x.is_cuda:
        return spec_ln_ref(x, w, b, eps, out_scale)
    nat = _nat()
    y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    rc = nat.lib().ab200_spec_ln(x.data_ptr(), x.stride(0), nat.ptr(w), nat.ptr(b), y.data_ptr(),
                                 y.stride(0), x.shape[0], x.shape[1], float(eps), float(out_scale),
                                 nat.stream_ptr())
    nat.check(rc, "spec_ln")
    launch_counter.add(1)
    return y


def mlp_spec_step(proj, emb, tok, emb_scale, ln_w, ln_b, eps=1e-6, tanh_approx=False):
    if not proj.is_cuda:
        return mlp_spec_step_ref(proj, emb, tok, emb_scale, ln_w, ln_b, eps, tanh_approx)
    nat = _nat()
    out = torch.empty(proj.shape, dtype=proj.dtype, device=proj.device)
    rc = nat.lib().ab200_mlp_spec_step(proj.data_ptr(), proj.stride(0), emb.data_ptr(),
                                       tok.data_ptr(), float(emb_scale), nat.ptr(ln_w),
                                       nat.ptr(ln_b), out.data_ptr(), out.stride(0), proj.shape[0],
                                       proj.shape[1], float(eps), int(tanh_approx), nat.stream_ptr())
    nat.check(rc, "mlp_spec_step")
    launch_counter.add(1)
    return out


def sum_lstm(gates, emb, tok, alpha, prev_c, w_cell, b_cell, w_state, b_state, eps=1e-6,
             tanh_approx=False):
    if not gates.is_cuda:
        return sum_lstm_ref(gates, emb, tok, alpha, prev_c, w_cell, b_cell, w_state, b_state, eps,
                            tanh_approx)
    nat = _nat()
    B, D4 = gates.shape
    D = D4 // 4
    c_out = torch.empty(B, D, dtype=gates.dtype, device=gates.device)
    h_out = torch.empty(B, D, dtype=gates.dtype, device=gates.device)
    rc = nat.lib().ab200_sum_lstm(
        gates.data_ptr(), gates.stride(0), emb.data_ptr(), emb.shape[1], tok.data_ptr(),
        float(alpha), nat.ptr(prev_c), prev_c.stride(0) if prev_c is not None else 0,
        nat.ptr(w_cell), nat.ptr(b_cell), nat.ptr(w_state), nat.ptr(b_state), c_out.data_ptr(),
        h_out.data_ptr(), D, B, D, float(eps), int(tanh_approx), nat.stream_ptr())
    nat.check(rc, "sum_lstm")
    launch_counter.add(1)
    return c_out, h_out


def verify_greedy(input_ids, target, row_start, num_draft, max_draft: int):
    """See ``verify_greedy_kernel``: returns (accepted int32 [R], next_tok int64 [R],
    sel_row int64 [R], out_tokens int64 [R, max_draft + 1])."""
    if not input_ids.is_cuda:
        return verify_greedy_ref(input_ids, target, row_start, num_draft, max_draft)
    nat = _nat()
    R = row_start.numel()
    dev = input_ids.device
    accepted = torch.empty(R, dtype=torch.int32, device=dev)
    next_tok = torch.empty(R, dtype=torch.int64, device=dev)
    sel_row = torch.empty(R, dtype=torch.int64, device=dev)
    out = torch.empty(R, max_draft + 1, dtype=torch.int64, device=dev)
    rc = nat.lib().ab200_verify_greedy(input_ids.data_ptr(), target.data_ptr(),
                                       row_start.data_ptr(), num_draft.data_ptr(), R, max_draft,
                                       accepted.data_ptr(), next_tok.data_ptr(), sel_row.data_ptr(),
                                       out.data_ptr(), nat.stream_ptr())
    nat.check(rc, "verify_greedy")
    launch_counter.add(1)
    return accepted, next_tok, sel_row, out
