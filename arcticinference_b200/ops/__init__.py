"""Tensor-level ops of the engine.

CUDA tensors always run the hand-written sm_100a kernels from ``_kernels.so``
(a missing or unloadable library raises -- there is no silent fallback on a
GPU). CPU tensors run the PyTorch restatements in :mod:`.reference`, which are
also the oracles of the numerics tests.
"""

from __future__ import annotations

import math
import sys
from dataclasses import dataclass, field

import numpy as np
import torch

from . import reference as ref

__all__ = [
    "linear", "linear_fp8", "linear_fp8_row", "quant_fp8", "quant_fp8_row", "gemm_nn", "embedding", "rmsnorm", "layernorm", "silu_mul", "silu_mul_blocked", "rope_cache",
    "gather_rows", "argmax_sample", "AttentionMetadata", "build_attention_metadata", "pick_tile_keys", "plan_attention_work",
    "attention", "attention_contiguous", "check_status", "count_launches", "launch_counter",
]


class _LaunchCounter:
    """Counts launches of this package's own kernels (used by bench.py). While an
    :class:`OpTimer` is active every counted op also drops a CUDA event, which attributes the
    device time since the previous op to the calling wrapper."""

    def __init__(self):
        self.n = 0
        self.timer = None

    def add(self, k: int = 1):
        self.n += k
        if self.timer is not None:
            self.timer.mark(sys._getframe(1).f_code.co_name)


class OpTimer:
    """Per-op device time of a stretch of eager execution.

        with ops.OpTimer() as t:
            model.forward(...)
        print(t.summary())

    An event follows every op; the time between consecutive events is booked on the later op
    (it includes that op's launch gap). ``head_start_us`` makes the GPU spin first so that the
    host can queue ahead and the gaps are the device's own, not Python's."""

    def __init__(self, head_start_us: float = 20000.0):
        self.head_start_us = head_start_us
        self.marks: list = []

    def __enter__(self):
        torch.cuda.synchronize()
        if self.head_start_us > 0:
            torch.cuda._sleep(int(self.head_start_us * 1900))
        self.mark("_start")
        launch_counter.timer = self
        return self

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, ev))

    def __exit__(self, *exc):
        launch_counter.timer = None
        torch.cuda.synchronize()

    def records(self) -> list:
        return [(n1, e0.elapsed_time(e1) * 1e3)
                for (n0, e0), (n1, e1) in zip(self.marks, self.marks[1:])]

    def summary(self) -> dict:
        out: dict = {}
        for name, us in self.records():
            tot, cnt = out.get(name, (0.0, 0))
            out[name] = (tot + us, cnt + 1)
        return dict(sorted(out.items(), key=lambda kv: -kv[1][0]))


launch_counter = _LaunchCounter()


def count_launches() -> int:
    return launch_counter.n


def _native():
    from . import native
    return native


def check_status(device=None):
    _native().check_status(device)


_ACT = {None: 0, "none": 0, "gelu": 1}


def quant_fp8(x: torch.Tensor):
    """bf16 [M, K] -> (e4m3 codes [M, K], scales fp32 [K/128, M]) per token and 128-wide k group."""
    from ..models import quant
    if not x.is_cuda:
        return quant.quant_activation_ref(x)
    nat = _native()
    M, K = x.shape
    xq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    sx_t = torch.empty(K // 128, M, dtype=torch.float32, device=x.device)
    rc = nat.lib().ab200_quant_fp8(x.data_ptr(), x.stride(0), xq.data_ptr(), xq.stride(0),
                                   sx_t.data_ptr(), sx_t.stride(0), M, K, nat.stream_ptr())
    nat.check(rc, "quant_fp8")
    launch_counter.add(1)
    return xq, sx_t


def quant_fp8_row(x: torch.Tensor, sync=None):
    """bf16 [M, K] -> ``QuantAct`` (e4m3 codes [M, K], one fp32 scale per token). ``sync``: a
    ``native.PeerSync`` whose wait part holds the kernel back until the ranks that store rows
    of ``x`` have signalled."""
    from ..models import quant
    if not x.is_cuda:
        return quant.quant_activation_row_ref(x)
    nat = _native()
    M, K = x.shape
    assert x.stride(1) == 1
    xq = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    sx = torch.empty(M, dtype=torch.float32, device=x.device)
    import ctypes
    rc = nat.lib().ab200_quant_fp8_row_wait(
        x.data_ptr(), x.stride(0), xq.data_ptr(), xq.stride(0), sx.data_ptr(), M, K,
        ctypes.byref(sync) if sync is not None else None,
        nat.status_buffer(x.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "quant_fp8_row")
    launch_counter.add(1)
    return quant.QuantAct(xq, sx)


# Storages of parameters (weights that no kernel of the compute stream writes). A linear layer
# whose weight lives in one of them requests its first weight tiles before it waits for the
# kernel launched before it, so the weight stream starts under that kernel's tail.
_static_storages: set = set()


def mark_static(t) -> None:
    """Declare ``t`` (a tensor or a quantised weight) a parameter. An in-place update of a
    parameter (a weight sync) is followed by other kernels before the next linear layer that
    reads it, which is what makes the early read safe."""
    if t is None:
        return
    q = getattr(t, "q", t)
    if isinstance(q, torch.Tensor) and q.is_cuda:
        _static_storages.add(q.untyped_storage().data_ptr())


def clear_static() -> None:
    _static_storages.clear()


def _is_static(t: torch.Tensor) -> bool:
    return bool(_static_storages) and t.untyped_storage().data_ptr() in _static_storages


def _linear_desc(x, ldx, sx, w, ldw, sw, out_ptr, ldo, M, N, K, bias, residual, act,
                 force_splits, peer, sync, device, w_tile_strides=None, w_static=False):
    """Fill an ``Ab200LinearDesc`` and launch it."""
    import ctypes
    nat = _native()
    ws = nat.workspace(device)
    d = nat.LinearDesc()
    d.x, d.ldx, d.sx = x, ldx, sx
    d.w, d.ldw, d.sw = w, ldw, sw
    d.out, d.ldo = out_ptr, ldo
    d.M, d.N, d.K = M, N, K
    d.bias = nat.ptr(bias)
    d.residual = nat.ptr(residual)
    d.ldr = residual.stride(0) if residual is not None else 0
    d.act = _ACT[act]
    d.workspace, d.workspace_bytes, d.force_splits = ws.data_ptr(), ws.numel(), force_splits
    if peer is not None:
        pp, world, pcols, poff, pldo = peer
        d.peer_ptrs = ctypes.cast(pp, ctypes.c_void_p)
        d.world, d.peer_cols, d.peer_row_off, d.ldo = world, pcols, poff, pldo
    if sync is not None:
        d.sync = sync
    if w_tile_strides is not None:
        d.w_tile_stride_n, d.w_tile_stride_k = w_tile_strides
    d.w_static = 1 if w_static else 0
    d.status = nat.status_buffer(device).data_ptr()
    rc = nat.lib().ab200_linear_desc(ctypes.byref(d), nat.stream_ptr())
    return rc


def linear_fp8_row(x, w, bias=None, residual=None, act=None, out=None, force_splits: int = 0,
                   peer=None, sync=None) -> torch.Tensor:
    """W8A8 fp8 linear with per-token activation scales and per-feature weight scales:
    ``x`` is a bf16 tensor (quantised here) or a ``QuantAct``; ``w`` an ``Fp8RowWeight``.
    ``peer`` = (ptr_array, world, peer_cols, row_off, ldo) scatters the output columns to the
    ranks' buffers (see ``ab200_linear_bf16_scatter``). ``sync`` (``native.PeerSync``): its
    wait part guards the first kernel that reads ``x``, its signal part is sent by the kernel
    that writes the output."""
    from ..models import quant
    if not w.is_cuda:
        y = quant.linear_fp8_row_ref(x, w, bias, residual, act)
        if out is not None:
            out.copy_(y)
            return out
        return y
    nat = _native()
    gemm_sync = sync
    if not isinstance(x, quant.QuantAct):
        xq = quant_fp8_row(x, sync=sync if (sync is not None and sync.wait_world > 0) else None)
        if sync is not None and sync.wait_world > 0:
            # the quantiser has waited; the GEMM only signals
            gemm_sync = nat.PeerSync.from_buffer_copy(sync)
            gemm_sync.wait_world = 0
    else:
        xq = x
    M, K = xq.q.shape
    N = w.shape[0]
    assert xq.q.stride(1) == 1 and K == w.shape[1]
    tile_strides = None
    if w.tiled:
        assert w.q.stride(3) == 1 and w.q.stride(2) == 128
        # (the stride of a dimension of size 1 is arbitrary: substitute the packed value)
        sk = w.q.stride(1) if w.q.shape[1] > 1 else 2048
        sn = w.q.stride(0) if w.q.shape[0] > 1 else sk * w.q.shape[1]
        tile_strides = (sn, sk)
        ldw = K
    else:
        assert w.q.stride(1) == 1
        ldw = w.q.stride(0)
    if peer is None:
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=w.device)
        assert out.stride(1) == 1
        out_ptr, ldo = out.data_ptr(), out.stride(0)
    else:
        out_ptr, ldo = None, peer[4]
    if M == 0:
        return out
    rc = _linear_desc(xq.q.data_ptr(), xq.q.stride(0), xq.scale.data_ptr(), w.q.data_ptr(),
                      ldw, w.scale.data_ptr(), out_ptr, ldo, M, N, K, bias, residual,
                      act, force_splits, peer, gemm_sync, w.device, tile_strides,
                      w_static=_is_static(w.q))
    nat.check(rc, "linear_fp8_row M=%d N=%d K=%d" % (M, N, K))
    launch_counter.add(1)
    return out


DEQUANT_MIN_TOKENS = 512
_dequant_scratch: dict = {}


def dequant_fp8(w) -> torch.Tensor:
    """The weight as a bf16 matrix: its resident shadow copy when the model keeps one, else
    expanded into a (per-device, reused) scratch matrix."""
    if getattr(w, "shadow", None) is not None:
        return w.shadow
    if not w.is_cuda:
        return w.dequantize()
    nat = _native()
    N, K = w.shape
    idx = w.device.index
    buf = _dequant_scratch.get(idx)
    if buf is None or buf.numel() < N * K:
        buf = torch.empty(max(N * K, 28672 * 4096), dtype=torch.bfloat16, device=w.device)
        _dequant_scratch[idx] = buf
    out = buf[:N * K].view(N, K)
    rc = nat.lib().ab200_dequant_fp8(w.q.data_ptr(), w.q.stride(0), w.scale.data_ptr(),
                                     w.scale.stride(0), out.data_ptr(), out.stride(0), N, K,
                                     nat.stream_ptr())
    nat.check(rc, "dequant_fp8")
    launch_counter.add(1)
    return out


W8A16_MAX_TOKENS = 128
W8A16_SHADOW_CROSSOVER = 64     # measured: above this the bf16 GEMM on a shadow copy is faster


def fp8_prefers_bf16(w, num_tokens: int) -> bool:
    """Which route a block-scaled fp8 linear takes for ``num_tokens`` rows. The weight-only
    kernel (fp8 bytes from HBM, expansion in the kernel) serves small steps: up to 64 tokens
    when the model keeps bf16 shadows (beyond that the expansion costs more than the bytes it
    saves: 105 us against 52 us for the gate/up projection at 128 tokens), up to 128 when it
    does not. Larger steps run the bf16 GEMM on the shadow, or on a copy expanded once per call
    when the step is long enough to amortise that; the W8A8 kernel covers what is left."""
    from ..models.quant import Fp8RowWeight
    if isinstance(w, Fp8RowWeight):
        return False
    shadow = getattr(w, "shadow", None) is not None
    if num_tokens <= (W8A16_SHADOW_CROSSOVER if shadow else W8A16_MAX_TOKENS):
        return False
    return shadow or num_tokens >= DEQUANT_MIN_TOKENS


def linear_fp8(x: torch.Tensor, w, out=None, force_splits: int = 0, peer=None,
               mode: str = "auto", sync=None) -> torch.Tensor:
    """Block-scaled fp8 linear: x bf16 [M, K] is quantised on the fly; w is an ``Fp8Weight``.
    ``peer`` = (ptr_array, world, peer_cols, row_off, ldo) scatters the output (see
    ``ab200_linear_bf16_scatter``)."""
    from ..models import quant
    if isinstance(w, quant.Fp8RowWeight):
        return linear_fp8_row(x, w, out=out, force_splits=force_splits, peer=peer, sync=sync)
    assert sync is None, "cross-rank ordering is not available for block-scaled fp8 linears"
    if isinstance(x, quant.QuantAct):
        x = x.dequantize()
    if not x.is_cuda:
        y = quant.linear_fp8_ref(x, w)
        if out is not None:
            out.copy_(y)
            return out
        return y
    nat = _native()
    M, K = x.shape
    N = w.shape[0]
    if peer is None and mode == "auto" and fp8_prefers_bf16(w, M):
        # bf16 GEMM on the shadow copy (or on a copy expanded once per long prefill step): the
        # activations stay in bf16 and the tensor cores never wait on per-block rescaling
        return linear(x, dequant_fp8(w), out=out)
    ws = nat.workspace(x.device)
    if peer is None:
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        out_ptr, ldo, pp, world, pcols, poff = out.data_ptr(), out.stride(0), None, 0, 0, 0
    else:
        pp, world, pcols, poff, ldo = peer
        out_ptr = None
    if M <= W8A16_MAX_TOKENS and mode != "w8a8":
        # decode: weight-only fp8, activations stay bf16, weights are expanded inside the kernel
        rc = nat.lib().ab200_linear_w8a16(
            x.data_ptr(), x.stride(0), w.q.data_ptr(), w.q.stride(0), w.scale.data_ptr(),
            w.scale.stride(0), out_ptr, ldo, M, N, K, ws.data_ptr(), ws.numel(), force_splits, pp,
            world, pcols, poff, nat.status_buffer(x.device).data_ptr(), nat.stream_ptr())
        nat.check(rc, "linear_w8a16 M=%d N=%d K=%d" % (M, N, K))
        launch_counter.add(1)
        return out
    xq, sx_t = quant_fp8(x)
    rc = nat.lib().ab200_linear_fp8(
        xq.data_ptr(), xq.stride(0), sx_t.data_ptr(), sx_t.stride(0), w.q.data_ptr(),
        w.q.stride(0), w.scale.data_ptr(), w.scale.stride(0), out_ptr, ldo, M, N, K,
        ws.data_ptr(), ws.numel(), force_splits, pp, world, pcols, poff,
        nat.status_buffer(x.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "linear_fp8 M=%d N=%d K=%d" % (M, N, K))
    launch_counter.add(1)
    return out


def linear(x: torch.Tensor, w, bias=None, residual=None, act=None, out=None,
           force_splits: int = 0, sync=None) -> torch.Tensor:
    """``out = act(x @ w.T + bias) + residual``; x [M, K] (row stride free), w [N, K] bf16 or
    an ``Fp8Weight``. ``sync``: optional ``native.PeerSync`` (wait for the ranks that produce
    ``x``, signal the ranks that consume ``out``)."""
    if not isinstance(w, torch.Tensor):
        from ..models.quant import Fp8RowWeight
        if isinstance(w, Fp8RowWeight):
            return linear_fp8_row(x, w, bias, residual, act, out=out, force_splits=force_splits,
                                  sync=sync)
        assert bias is None and residual is None and act is None
        return linear_fp8(x, w, out=out, force_splits=force_splits, sync=sync)
    if not isinstance(x, torch.Tensor):   # a quantised activation meeting a bf16 weight
        x = x.dequantize()
    if not x.is_cuda:
        y = ref.linear(x, w, bias, residual, act)
        if out is not None:
            out.copy_(y)
            return out
        return y
    nat = _native()
    L = nat.lib()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    assert out.stride(1) == 1
    if M == 0:
        return out
    static = _is_static(w)
    if sync is not None or static:
        rc = _linear_desc(x.data_ptr(), x.stride(0), None, w.data_ptr(), w.stride(0), None,
                          out.data_ptr(), out.stride(0), M, N, K, bias, residual, act,
                          force_splits, None, sync, x.device, w_static=static)
        nat.check(rc, "linear_bf16 M=%d N=%d K=%d" % (M, N, K))
        launch_counter.add(1)
        return out
    ws = nat.workspace(x.device)
    rc = L.ab200_linear_bf16(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
        M, N, K, nat.ptr(bias), nat.ptr(residual),
        residual.stride(0) if residual is not None else 0, _ACT[act],
        ws.data_ptr(), ws.numel(), force_splits, nat.status_buffer(x.device).data_ptr(),
        nat.stream_ptr())
    nat.check(rc, "linear_bf16 M=%d N=%d K=%d" % (M, N, K))
    launch_counter.add(1)
    return out


def gemm_nn(x: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
    """``x @ wt`` with wt [K, N] row-major (MN-major B operand path)."""
    if not x.is_cuda:
        return (x.float() @ wt.float()).to(x.dtype)
    nat = _native()
    M, K = x.shape
    N = wt.shape[1]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    rc = nat.lib().ab200_gemm_bf16_nn(x.data_ptr(), x.stride(0), wt.data_ptr(), wt.stride(0),
                                      out.data_ptr(), out.stride(0), M, N, K,
                                      nat.status_buffer(x.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "gemm_bf16_nn")
    launch_counter.add(1)
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0, out=None):
    if not table.is_cuda:
        return ref.embedding(ids, table, vocab_start)
    nat = _native()
    ids = ids.to(torch.int64).contiguous()
    T, H = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = nat.lib().ab200_embedding(ids.data_ptr(), table.data_ptr(), out.data_ptr(), T, H,
                                   table.shape[0], vocab_start, nat.stream_ptr())
    nat.check(rc, "embedding")
    launch_counter.add(1)
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual=None, out=None,
            quant: bool = False):
    """y = RMSNorm(x (+ residual)); ``residual`` (contiguous) is updated in place. With
    ``quant`` the result is a ``QuantAct`` (e4m3 rows with one scale per token, produced in the
    same pass) for an fp8 linear layer."""
    if not x.is_cuda:
        y = ref.rmsnorm(x, weight, eps, residual)
        if quant:
            from ..models.quant import quant_activation_row_ref
            return quant_activation_row_ref(y)
        if out is not None:
            out.copy_(y)
            return out
        return y
    nat = _native()
    T, H = x.shape
    if quant:
        from ..models.quant import QuantAct
        if residual is not None:
            assert residual.is_contiguous()
        yq = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=x.device)
        sy = torch.empty(T, dtype=torch.float32, device=x.device)
        rc = nat.lib().ab200_rmsnorm_quant(x.data_ptr(), x.stride(0), nat.ptr(residual),
                                           weight.data_ptr(), yq.data_ptr(), yq.stride(0),
                                           sy.data_ptr(), None, 0, T, H, float(eps),
                                           nat.stream_ptr())
        nat.check(rc, "rmsnorm_quant")
        launch_counter.add(1)
        return QuantAct(yq, sy)
    if out is None:
        out = torch.empty(T, H, dtype=x.dtype, device=x.device)
    if residual is not None:
        assert residual.is_contiguous()
    rc = nat.lib().ab200_rmsnorm(x.data_ptr(), x.stride(0), nat.ptr(residual), weight.data_ptr(),
                                 out.data_ptr(), out.stride(0), T, H, float(eps), nat.stream_ptr())
    nat.check(rc, "rmsnorm")
    launch_counter.add(1)
    return out


def layernorm(x, gamma, beta, eps: float, residual=None):
    if not x.is_cuda:
        return ref.layernorm(x, gamma, beta, eps, residual)
    nat = _native()
    x = x.contiguous()
    T, H = x.shape
    out = torch.empty_like(x)
    if residual is not None:
        residual = residual.contiguous()
    rc = nat.lib().ab200_layernorm(x.data_ptr(), nat.ptr(residual), gamma.data_ptr(),
                                   beta.data_ptr(), out.data_ptr(), T, H, float(eps),
                                   nat.stream_ptr())
    nat.check(rc, "layernorm")
    launch_counter.add(1)
    return out


def silu_mul_blocked(x: torch.Tensor, nblk: int = 1, out=None, quant: bool = False):
    """x: [T, nblk * 2 * I] as nblk blocks of (gate | up) -> [T, nblk * I]; with ``quant`` a
    ``QuantAct`` of the same values (one scale per token over the whole output row)."""
    if not x.is_cuda:
        y = ref.silu_mul_blocked(x, nblk)
        if quant:
            from ..models.quant import quant_activation_row_ref
            return quant_activation_row_ref(y)
        return y
    nat = _native()
    assert x.is_contiguous()
    T, width = x.shape
    inter = width // (2 * nblk)
    if quant:
        from ..models.quant import QuantAct
        oq = torch.empty(T, nblk * inter, dtype=torch.float8_e4m3fn, device=x.device)
        so = torch.empty(T, dtype=torch.float32, device=x.device)
        rc = nat.lib().ab200_silu_mul_quant(x.data_ptr(), oq.data_ptr(), oq.stride(0),
                                            so.data_ptr(), T, inter, nblk, nat.stream_ptr())
        nat.check(rc, "silu_mul_quant")
        launch_counter.add(1)
        return QuantAct(oq, so)
    if out is None:
        out = torch.empty(T, nblk * inter, dtype=x.dtype, device=x.device)
    rc = nat.lib().ab200_silu_mul(x.data_ptr(), out.data_ptr(), T, inter, nblk, nat.stream_ptr())
    nat.check(rc, "silu_mul")
    launch_counter.add(1)
    return out


def silu_mul(x: torch.Tensor, out=None):
    return silu_mul_blocked(x, 1, out)


def rope_cache(qkv, positions, slots, inv_freq, k_cache, v_cache, Hq, Hkv, D, rotate_q=True,
               sync=None):
    """In-place neox RoPE on the q and k parts of ``qkv`` [T, (Hq+2Hkv)*D] and write of the
    rotated k and of v into the paged caches [num_blocks, Hkv, block_size, D]."""
    if not qkv.is_cuda:
        return ref.rope_cache(qkv, positions, slots, inv_freq, k_cache, v_cache, Hq, Hkv, D,
                              rotate_q)
    nat = _native()
    T = qkv.shape[0]
    bs = k_cache.shape[2]
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    assert positions.dtype == torch.int64 and (slots is None or slots.dtype == torch.int64)
    import ctypes
    rc = nat.lib().ab200_rope_cache_wait(
        qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), nat.ptr(slots), inv_freq.data_ptr(),
        k_cache.data_ptr(), v_cache.data_ptr(), T, Hq, Hkv, D, bs, k_cache.shape[0] * bs,
        1 if rotate_q else 0, ctypes.byref(sync) if sync is not None else None,
        nat.status_buffer(qkv.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "rope_cache")
    launch_counter.add(1)


def qk_norm(qkv, wq, wk, Hq, Hkv, D, eps: float, sync=None):
    """In-place RMSNorm over head_dim of the ``Hq`` query and ``Hkv`` key heads of every row of
    ``qkv`` [T, (Hq + 2*Hkv) * D] (the value heads stay as they are); ``wq`` / ``wk`` [D] are
    shared by the heads. Runs between the QKV projection and RoPE in Qwen3. ``sync``: wait for
    the ranks that store rows of ``qkv`` before reading it."""
    if not qkv.is_cuda:
        return ref.qk_norm(qkv, wq, wk, Hq, Hkv, D, eps)
    nat = _native()
    import ctypes
    assert wq.is_contiguous() and (wk is None or wk.is_contiguous())
    rc = nat.lib().ab200_qk_norm(qkv.data_ptr(), qkv.stride(0), wq.data_ptr(), nat.ptr(wk),
                                 qkv.shape[0], Hq, Hkv, D, float(eps),
                                 ctypes.byref(sync) if sync is not None else None,
                                 nat.status_buffer(qkv.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "qk_norm")
    launch_counter.add(1)
    return qkv


def peer_barrier(flag_arrays, my_rank: int, epoch_counter: torch.Tensor, limit_ms: int = 1000) -> None:
    """Flag barrier among ``len(flag_arrays)`` ranks with a bounded wait. ``flag_arrays[r]`` is
    rank r's array of uint32 arrival slots (int32 tensors of >= 16 elements, here or in peer
    memory); ``epoch_counter`` is this rank's int32[1] barrier count. A peer that does not
    arrive within ``limit_ms`` leaves code 2 in the status word (``check_status`` raises
    ``KernelTimeout``); nothing hangs."""
    import ctypes
    nat = _native()
    arr = (ctypes.c_void_p * len(flag_arrays))(*[t.data_ptr() for t in flag_arrays])
    nat.declare("ab200_barrier_timed", ctypes.c_int,
                [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                 ctypes.c_void_p, ctypes.c_void_p])
    rc = nat.lib().ab200_barrier_timed(arr, my_rank, len(flag_arrays), epoch_counter.data_ptr(),
                                       int(limit_ms), nat.status_buffer(epoch_counter.device).data_ptr(),
                                       nat.stream_ptr())
    nat.check(rc, "barrier_timed")
    launch_counter.add(1)


POOL_MODES = {"cls": 0, "mean": 1, "last": 2}


def bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps: float):
    """LayerNorm(word[ids] + pos[positions] + typ[type_ids]) in one pass. ids/positions/type_ids
    int64 [T] (type_ids may be None = all zero)."""
    if not word.is_cuda:
        return ref.bert_embed_ln(ids, positions, type_ids, word, pos, typ, gamma, beta, eps)
    nat = _native()
    T, H = ids.numel(), word.shape[1]
    out = torch.empty(T, H, dtype=word.dtype, device=word.device)
    rc = nat.lib().ab200_bert_embed_ln(
        ids.data_ptr(), positions.data_ptr(), nat.ptr(type_ids), word.data_ptr(), pos.data_ptr(),
        typ.data_ptr(), gamma.data_ptr(), beta.data_ptr(), out.data_ptr(), T, H, word.shape[0],
        pos.shape[0], typ.shape[0], float(eps), nat.status_buffer(word.device).data_ptr(),
        nat.stream_ptr())
    nat.check(rc, "bert_embed_ln")
    launch_counter.add(1)
    return out


def pool_normalize(h, starts, mode: str = "cls", normalize: bool = True, out=None):
    """Per-sequence pooling of h [T, H] (sequence i owns rows starts[i]:starts[i+1]; ``starts``
    int64 [S+1] on h's device) and optional L2 normalisation. Returns fp32 [S, H]."""
    if not h.is_cuda:
        return ref.pool_normalize(h, starts, mode, normalize)
    nat = _native()
    S, H = starts.numel() - 1, h.shape[1]
    if out is None:
        out = torch.empty(S, H, dtype=torch.float32, device=h.device)
    rc = nat.lib().ab200_pool_normalize(h.data_ptr(), h.stride(0), starts.data_ptr(),
                                        out.data_ptr(), S, H, POOL_MODES[mode],
                                        1 if normalize else 0, nat.stream_ptr())
    nat.check(rc, "pool_normalize")
    launch_counter.add(1)
    return out


def kv_bulk_write(kv_all, positions, slots, inv_freq, k_caches, v_caches, Hkv, D, tables=None,
                  k_scales=None, v_scales=None):
    """RoPE on K and paged-cache write of K and V for several layers in one launch.
    ``kv_all`` [T, L*2*Hkv*D] holds layer j at columns j*2*Hkv*D (K heads, then V heads);
    ``k_caches / v_caches`` are the L cache tensors [num_blocks, Hkv, block_size, D] (bf16, or
    float8_e4m3fn together with fp32 ``k_scales / v_scales`` [L]). ``tables`` = (k_ptrs, v_ptrs)
    int64 device tensors of the cache base addresses, built once by the caller."""
    if not kv_all.is_cuda:
        return ref.kv_bulk_write(kv_all, positions, slots, inv_freq, k_caches, v_caches, Hkv, D,
                                 k_scales, v_scales)
    nat = _native()
    L = len(k_caches)
    T = kv_all.shape[0]
    if tables is None:
        tables = (torch.tensor([c.data_ptr() for c in k_caches], dtype=torch.int64, device=kv_all.device),
                  torch.tensor([c.data_ptr() for c in v_caches], dtype=torch.int64, device=kv_all.device))
    fp8 = k_caches[0].dtype == torch.float8_e4m3fn
    bs = k_caches[0].shape[2]
    assert kv_all.shape[1] == L * 2 * Hkv * D and slots.dtype == torch.int64
    rc = nat.lib().ab200_kv_bulk_write(
        kv_all.data_ptr(), kv_all.stride(0), positions.data_ptr(), slots.data_ptr(),
        inv_freq.data_ptr(), tables[0].data_ptr(), tables[1].data_ptr(), nat.ptr(k_scales),
        nat.ptr(v_scales), T, L, Hkv, D, bs, k_caches[0].shape[0] * bs, 1 if fp8 else 0,
        nat.status_buffer(kv_all.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "kv_bulk_write")
    launch_counter.add(1)


def kv_write_fp4(k, v, slots, k_codes, v_codes, k_scales, v_scales, Hkv, D):
    """NVFP4 cache write of one layer: k, v bf16 [T, Hkv*D] -> e2m1 codes [num_blocks, Hkv,
    block_size, D/2] uint8 and e4m3 group scales [num_blocks, Hkv, block_size, D/16] uint8."""
    bs = k_codes.shape[2]
    if not k.is_cuda:
        ok = slots >= 0
        s = slots[ok]
        blk, off = s // bs, s % bs
        T = k.shape[0]
        for src, codes, scales in ((k, k_codes, k_scales), (v, v_codes, v_scales)):
            c, sc, _ = ref.quantize_nvfp4(src.reshape(T, Hkv, D))
            codes[blk, :, off] = c[ok]
            scales[blk, :, off] = sc[ok]
        return
    nat = _native()
    rc = nat.lib().ab200_kv_write_fp4(
        k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), slots.data_ptr(),
        k_codes.data_ptr(), v_codes.data_ptr(), k_scales.data_ptr(), v_scales.data_ptr(),
        k.shape[0], Hkv, D, bs, k_codes.shape[0] * bs,
        nat.status_buffer(k.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "kv_write_fp4")
    launch_counter.add(1)


def kv_read_fp4(codes, scales, slots, Hkv, D):
    """Rows of an NVFP4 cache tensor at ``slots`` expanded to bf16 [R, Hkv*D]."""
    bs = codes.shape[2]
    R = slots.numel()
    if not codes.is_cuda:
        blk, off = slots // bs, slots % bs
        c = codes[blk, :, off].long()
        vals = torch.tensor(ref.E2M1_VALUES, dtype=torch.float32)
        nib = torch.stack([c & 15, c >> 4], -1).reshape(R, Hkv, D)
        x = vals[nib & 7] * torch.where((nib & 8) > 0, -1.0, 1.0)
        s = scales[blk, :, off].view(torch.float8_e4m3fn).float().repeat_interleave(16, -1)
        return (x * s).reshape(R, Hkv * D).to(torch.bfloat16)
    nat = _native()
    out = torch.empty(R, Hkv * D, dtype=torch.bfloat16, device=codes.device)
    rc = nat.lib().ab200_kv_read_fp4(codes.data_ptr(), scales.data_ptr(), slots.data_ptr(),
                                     out.data_ptr(), out.stride(0), R, Hkv, D, bs,
                                     nat.stream_ptr())
    nat.check(rc, "kv_read_fp4")
    launch_counter.add(1)
    return out


def gather_rows(src: torch.Tensor, idx: torch.Tensor, out=None):
    if not src.is_cuda:
        return ref.gather_rows(src, idx)
    nat = _native()
    R, H = idx.numel(), src.shape[1]
    if out is None:
        out = torch.empty(R, H, dtype=src.dtype, device=src.device)
    rc = nat.lib().ab200_gather_rows(src.data_ptr(), src.stride(0), idx.data_ptr(), out.data_ptr(),
                                     R, H, nat.stream_ptr())
    nat.check(rc, "gather_rows")
    launch_counter.add(1)
    return out


def patch_ids(ids: torch.Tensor, src_rows: torch.Tensor, prev_ids: torch.Tensor) -> None:
    """In place: ``ids[i] = prev_ids[src_rows[i]]`` where ``src_rows[i] >= 0`` (all int64)."""
    if not ids.is_cuda:
        m = src_rows >= 0
        ids[m] = prev_ids[src_rows[m]]
        return
    nat = _native()
    rc = nat.lib().ab200_patch_ids(ids.data_ptr(), src_rows.data_ptr(), prev_ids.data_ptr(),
                                   ids.numel(), prev_ids.numel(), nat.stream_ptr())
    nat.check(rc, "patch_ids")
    launch_counter.add(1)


def argmax_sample(logits: torch.Tensor, temperature=None, seeds=None, index_offset: int = 0,
                  out_ids=None, out_vals=None):
    """Row-wise token choice: arg-max where temperature <= 0, else an exact softmax sample
    (Gumbel-max). Returns (ids int64 [B], best value fp32 [B])."""
    if not logits.is_cuda:
        return ref.argmax_sample(logits, temperature, seeds, index_offset)
    nat = _native()
    B, V = logits.shape
    assert logits.stride(1) == 1
    if out_ids is None:
        out_ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    if out_vals is None:
        out_vals = torch.empty(B, dtype=torch.float32, device=logits.device)
    dt = 0 if logits.dtype == torch.bfloat16 else 1
    assert logits.dtype in (torch.bfloat16, torch.float32)
    rc = nat.lib().ab200_argmax_sample(logits.data_ptr(), dt, logits.stride(0), B, V,
                                       nat.ptr(temperature), nat.ptr(seeds), out_ids.data_ptr(),
                                       out_vals.data_ptr(), index_offset, nat.stream_ptr())
    nat.check(rc, "argmax_sample")
    launch_counter.add(1)
    return out_ids, out_vals


def topk_topp_mask(logits: torch.Tensor, temperature=None, top_k=None, top_p=None):
    """fp32 [B, V]: ``logits / temperature`` for the tokens of each row's top-k / top-p set and
    -inf for the rest, ready for :func:`argmax_sample` (no sort, no probability vector).
    temperature fp32 [B]; top_k int64 [B] (<= 0: off); top_p fp32 [B] (>= 1: off). Tokens with
    equal logits stay or go together."""
    if not logits.is_cuda:
        return ref.topk_topp_mask(logits, temperature, top_k, top_p)
    nat = _native()
    x = logits if logits.dtype == torch.float32 else logits.float()
    assert x.stride(1) == 1
    B, V = x.shape
    out = torch.empty(B, V, dtype=torch.float32, device=x.device)
    for t, dt in ((temperature, torch.float32), (top_k, torch.int64), (top_p, torch.float32)):
        assert t is None or (t.dtype == dt and t.is_contiguous() and t.numel() == B)
    rc = nat.lib().ab200_topk_topp_mask(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0),
                                        B, V, nat.ptr(temperature), nat.ptr(top_k),
                                        nat.ptr(top_p), nat.stream_ptr())
    nat.check(rc, "topk_topp_mask")
    launch_counter.add(1)
    return out


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
TILE_KEYS = 128


@dataclass
class AttentionMetadata:
    """Host-built description of one attention call (shared by all layers of a step).

    ``work`` is the [num_work, 8] int32 table consumed by the kernel
    (csrc/attention.cu): one entry per (query tile, KV split)."""
    q_lens: list
    kv_lens: list
    num_tokens: int
    work: torch.Tensor | None = None
    tok_splits: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None
    max_splits: int = 1
    num_work: int = 0
    o_part: torch.Tensor | None = None
    lse_part: torch.Tensor | None = None
    tile_keys: int = 128     # 64 for decode-shaped calls (few query rows per sequence)
    extra: dict = field(default_factory=dict)


def plan_attention_work(q_lens, kv_lens, G: int, causal: bool = True, num_sms: int = 148,
                        Hkv: int = 1, seq_rows=None, allow_split: bool = True,
                        max_splits_cap: int = 16):
    """Pure-host planner. Returns (work [n,8] int32 ndarray, tok_splits [T] int32, max_splits).

    Query tokens of a sequence are cut into tiles of 128/G tokens. When the call has too few
    tiles to occupy the GPU (decode), the keys of each sequence are cut into up to 16 splits
    of whole 128-key tiles."""
    tpt = 128 // G
    if len(q_lens) >= 16 and max(q_lens) == 1 and min(q_lens) == 1:
        return _plan_decode_work(kv_lens, G, causal, num_sms, Hkv, seq_rows, allow_split,
                                 max_splits_cap)
    rows = []
    T = int(sum(q_lens))
    tok_splits = np.ones(max(T, 1), dtype=np.int32)
    n_tiles_total = sum((ql + tpt - 1) // tpt for ql in q_lens)
    if q_lens and max(q_lens) * G <= 32:
        num_sms *= 2  # decode-shaped calls run two CTAs per SM (64-key tiles)
    t0 = 0
    max_splits = 1
    for i, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        if ql <= 0:
            continue
        seq_field = i if seq_rows is None else int(seq_rows[i])
        key_tiles = (kl + TILE_KEYS - 1) // TILE_KEYS
        ns = 1
        if allow_split and n_tiles_total * Hkv < num_sms and key_tiles > 4:
            want = max(1, num_sms // max(1, n_tiles_total * Hkv))
            ns = int(min(16, max_splits_cap, want, max(1, key_tiles // 2)))
        tiles_per_split = (key_tiles + ns - 1) // ns
        ns = (key_tiles + tiles_per_split - 1) // tiles_per_split
        max_splits = max(max_splits, ns)
        for a in range(0, ql, tpt):
            n = min(tpt, ql - a)
            q_pos0 = kl - ql + a
            for s in range(ns):
                ks = s * tiles_per_split * TILE_KEYS
                ke = min(kl, (s + 1) * tiles_per_split * TILE_KEYS)
                rows.append((seq_field, t0 + a, n, q_pos0, ks, ke, s, ns))
        if ns > 1:
            tok_splits[t0:t0 + ql] = ns
        t0 += ql
    if causal:
        # heaviest tiles first: later query tiles see more keys
        rows.sort(key=lambda r: -(min(r[5], r[3] + r[2]) - r[4]))
    work = np.asarray(rows, dtype=np.int32).reshape(-1, 8)
    return work, tok_splits, max_splits


def tail_split_plan(n_seqs: int, Hkv: int, slots: int, max_splits: int = 4):
    """Decode call with more CTAs (sequences x KV heads) than the GPU holds at once: the CTAs
    run in waves of ``slots``, all of about the same length, and the last wave is partly
    empty (1024 CTAs on 296 slots: three full waves and 136 CTAs in a fourth). Returns
    (number of sequences to cut, pieces per cut sequence): the sequences of that last wave
    are cut so that their pieces cover all slots, e.g. 17 sequences in 2 pieces each; with the
    pieces placed last in the work list the call takes 3.5 waves instead of 4. (Cutting
    every sequence instead measured no gain: every CTA then pays its set-up twice.)"""
    ctas = n_seqs * Hkv
    full, rem = divmod(ctas, slots)
    if full < 1 or rem == 0 or rem > 0.7 * slots:
        return 0, 1
    pieces = int(min(max_splits, max(2, round(slots / float(rem)))))
    return -(-rem // Hkv), pieces


def _plan_decode_work(kv_lens, G, causal, num_sms, Hkv, seq_rows, allow_split, max_splits_cap):
    """The planner above for the one-token-per-sequence case, on arrays (same rows, same
    order): a serving step with a thousand sequences must not spend milliseconds here."""
    kl = np.asarray(kv_lens, dtype=np.int64)
    R = kl.size
    if G <= 32:
        num_sms *= 2
    key_tiles = (kl + TILE_KEYS - 1) // TILE_KEYS
    ns = np.ones(R, dtype=np.int64)
    if allow_split and R * Hkv < num_sms:
        want = max(1, num_sms // max(1, R * Hkv))
        cand = np.minimum(np.minimum(16, max_splits_cap), np.minimum(want, np.maximum(1, key_tiles // 2)))
        ns = np.where(key_tiles > 4, cand, 1)
    elif allow_split and max_splits_cap > 1:
        n_cut, pieces = tail_split_plan(R, Hkv, num_sms, int(min(4, max_splits_cap)))
        if n_cut > 0:
            # the longest sequences are cut (at least 4 tiles per piece)
            longest = np.argsort(-kl, kind="stable")[:n_cut]
            longest = longest[key_tiles[longest] >= 4 * pieces]
            ns[longest] = pieces
    tps = (key_tiles + ns - 1) // ns
    ns = (key_tiles + tps - 1) // tps
    seq = np.arange(R, dtype=np.int64) if seq_rows is None else np.asarray(seq_rows, dtype=np.int64)
    rep = np.repeat(np.arange(R), ns)
    first = np.cumsum(ns) - ns
    sidx = np.arange(rep.size) - first[rep]                     # split index within its sequence
    ks = sidx * tps[rep] * TILE_KEYS
    ke = np.minimum(kl[rep], (sidx + 1) * tps[rep] * TILE_KEYS)
    work = np.stack([seq[rep], rep, np.ones_like(rep), kl[rep] - 1, ks, ke, sidx, ns[rep]], 1)
    if causal:
        order = np.argsort(-(np.minimum(ke, kl[rep]) - ks), kind="stable")
        work = work[order]
    tok_splits = ns.astype(np.int32)
    return work.astype(np.int32), tok_splits, int(ns.max()) if R else 1


def upload(a: np.ndarray, device) -> torch.Tensor:
    """Host array -> device tensor without stalling the host. A copy from pageable memory
    makes the host wait until the stream has reached it, i.e. until every step queued before
    it has finished, which would undo run-ahead stepping; so the array goes through pinned
    memory of the caching host allocator (kept alive until the copy has run)."""
    t = torch.from_numpy(a)
    dev = torch.device(device)
    if dev.type == "cuda":
        t = t.pin_memory()
    return t.to(dev, non_blocking=True)


def pick_tile_keys(q_lens, G: int) -> int:
    """64-key tiles when every sequence's query rows fit one warp of the 128-row tile."""
    return 64 if q_lens and max(q_lens) * G <= 32 else 128


def build_attention_metadata(q_lens, kv_lens, block_tables, G, Hq, D, device, causal=True,
                             Hkv=None, seq_rows=None, allow_split=True,
                             work_capacity: int | None = None) -> AttentionMetadata:
    Hkv = Hkv if Hkv is not None else Hq // G
    work, tok_splits, max_splits = plan_attention_work(q_lens, kv_lens, G, causal, Hkv=Hkv,
                                                       seq_rows=seq_rows, allow_split=allow_split)
    T = int(sum(q_lens))
    n = work.shape[0]
    if work_capacity is not None:
        assert n <= work_capacity
        pad = np.zeros((work_capacity - n, 8), dtype=np.int32)
        work = np.concatenate([work, pad], 0)
    meta = AttentionMetadata(list(q_lens), list(kv_lens), T)
    dev = torch.device(device)
    meta.work = upload(work, dev)
    meta.tok_splits = upload(tok_splits, dev)
    meta.block_tables = block_tables
    meta.max_splits = max_splits
    meta.num_work = work.shape[0]
    meta.tile_keys = pick_tile_keys(q_lens, G)
    if max_splits > 1 and dev.type == "cuda":
        meta.o_part = torch.empty(max_splits, T, Hq, D, dtype=torch.float32, device=dev)
        meta.lse_part = torch.empty(max_splits, T, Hq, dtype=torch.float32, device=dev)
    return meta


def attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              meta: AttentionMetadata, Hq: int, Hkv: int, D: int, scale: float | None = None,
              causal: bool = True, out=None, lse_out=None):
    """Paged attention. q: [T, Hq*D] (row stride free); caches [num_blocks, Hkv, block_size, D];
    ``meta.block_tables`` int32 [num_seqs, max_blocks]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    T = q.shape[0]
    if not q.is_cuda:
        o, lse = ref.attention(q, k_cache, v_cache, meta.block_tables, meta.q_lens, meta.kv_lens,
                               Hq, Hkv, D, scale, causal, return_lse=True)
        if lse_out is not None:
            lse_out.copy_(lse)
        if out is not None:
            out.copy_(o)
            return out
        return o
    nat = _native()
    if out is None:
        out = torch.empty(T, Hq * D, dtype=q.dtype, device=q.device)
    bt = meta.block_tables
    assert bt.dtype == torch.int32 and bt.is_contiguous()
    assert k_cache.is_contiguous() and v_cache.is_contiguous()
    rc = nat.lib().ab200_attention(
        q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), 0, k_cache.shape[0],
        k_cache.shape[2], bt.data_ptr(), bt.shape[1], meta.work.data_ptr(), meta.num_work,
        nat.ptr(meta.tok_splits), meta.max_splits, T, Hq, Hkv, D, 1 if causal else 0,
        float(scale), out.data_ptr(), out.stride(0), nat.ptr(meta.o_part), nat.ptr(meta.lse_part),
        nat.ptr(lse_out), meta.tile_keys, nat.status_buffer(q.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "attention")
    launch_counter.add(2 if meta.max_splits > 1 else 1)
    return out


def attention_contiguous(q, k, v, seq_lens, H: int, D: int, scale: float | None = None,
                         causal: bool = False, meta: AttentionMetadata | None = None, out=None):
    """Varlen attention over packed sequences whose K/V rows are contiguous (encoder path).
    q, k, v: [T, H*D] views with a common row stride (e.g. slices of a fused qkv buffer)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return ref.attention_contiguous(q, k, v, seq_lens, H, D, scale, causal)
    nat = _native()
    T = q.shape[0]
    if meta is None:
        starts = np.concatenate([[0], np.cumsum(seq_lens)[:-1]]).astype(np.int64)
        meta = build_attention_metadata(seq_lens, seq_lens, None, 1, H, D, q.device, causal=causal,
                                        Hkv=H, seq_rows=starts, allow_split=False)
    if out is None:
        out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
    assert k.stride(0) == v.stride(0)
    rc = nat.lib().ab200_attention(
        q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), k.stride(0), T, 0, None, 0,
        meta.work.data_ptr(), meta.num_work, None, 1, T, H, H, D, 1 if causal else 0, float(scale),
        out.data_ptr(), out.stride(0), None, None, None, 128,
        nat.status_buffer(q.device).data_ptr(), nat.stream_ptr())
    nat.check(rc, "attention_contiguous")
    launch_counter.add(1)
    return out
