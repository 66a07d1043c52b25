"""Collectives fused into the compute kernels over NVLink peer memory.

Every rank allocates one symmetric heap (``torch.distributed._symmetric_memory``)
that all ranks map. The hot exchanges then happen inside the kernels:

* sequence -> head exchange (the reference's first ``all_to_all_single``,
  arctic_inference/vllm/ulysses.py:436-438): the QKV projection GEMM's epilogue
  stores each head block's columns directly into the owning rank's ``qkv`` buffer
  (``ab200_linear_bf16_scatter``), rows in global token order;
* head -> sequence exchange (ulysses.py:450-455): the attention kernel's epilogue
  stores each token's output row into the buffer of the rank that owns the token
  (``ab200_attention_scatter``); the o_proj GEMM then reads local memory only;
* tensor-parallel reductions of shift mode: the row-parallel GEMM writes its
  partial product into the heap; small reductions run ``ab200_allreduce`` (every rank sums
  all ranks' partials with peer loads), large ones ``ab200_allreduce2`` (one launch: each
  rank reduces its slice by peer loads and stores the result into every rank's buffer, so
  (W-1)/W of the tensor crosses NVLink per direction instead of W-1 times the tensor; it
  costs two flag exchanges, so the switch-over size falls with the number of ranks).
  Both accumulate in fp32 in rank order, so all ranks get the same bits.

Producer and consumer kernels order themselves across ranks without a kernel in between: the
last block of a producer (scatter GEMM, scatter attention, row-parallel GEMM) signals every
rank, and the first kernel that reads the data (RoPE + cache write, the activation quantiser or
the o_proj GEMM's load warp, the fused reduce + RMSNorm) waits for the W signals
(``csrc/common/peer.cuh``; bounded waits). ``ab200_barrier`` (a symmetric flag exchange) remains
for the row gathers. All loads of remote data are plain peer loads or TMA loads from *local*
memory; nothing here uses cluster-multicast loads.

Small tensor-parallel reductions are folded into the RMSNorm that follows them
(``ab200_reduce_rmsnorm``): GEMM -> reduce+norm(+fp8 quantisation) is two launches where the
unfused path has four (GEMM, barrier, all-reduce, norm).

Supported shapes of the rank grid: TP=1 x SP=N (with or without shift) and TP=N x
SP=1. TP x SP grids with both > 1 use the library-collective communicator.
"""

from __future__ import annotations

import ctypes
import logging
import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops import native
from .comm import Communicator

logger = logging.getLogger(__name__)

_ALIGN = 1 << 12


def _ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


class PendingReduce:
    """A row-parallel product whose partial sums sit in the ranks' heaps, to be reduced by the
    kernel that consumes it (``FusedCommunicator.reduce_rmsnorm`` / ``realize``)."""

    __slots__ = ("key", "rows", "cols")

    def __init__(self, key: int, rows: int, cols: int):
        self.key, self.rows, self.cols = key, rows, cols

    @property
    def shape(self):
        return (self.rows, self.cols)


class _Channel:
    """Arrival words and counters of one kind of exchange (see ``TailSignal`` / ``PeerWait``)."""

    BYTES = 256

    def __init__(self, peer_base, offset: int, rank: int, world: int):
        self.flag_ptrs = _ptr_array([b + offset for b in peer_base])
        base = peer_base[rank] + offset
        self.flags, self.done, self.epoch = base, base + 128, base + 192
        self.rank, self.world = rank, world

    def sync(self, signal: bool = False, wait: bool = False) -> "native.PeerSync":
        s = native.PeerSync()
        if signal:
            s.sig_flag_ptrs = ctypes.cast(self.flag_ptrs, ctypes.c_void_p)
            s.sig_done_ctr, s.sig_epoch_ctr = self.done, self.epoch
            s.sig_rank, s.sig_world = self.rank, self.world
        if wait:
            s.wait_flags, s.wait_epoch_ctr, s.wait_world = self.flags, self.epoch, self.world
        return s


class FusedCommunicator(Communicator):
    fused = True

    def __init__(self, tp: int, sp: int, device: torch.device):
        super().__init__(tp, sp, device)
        if tp > 1 and sp > 1:
            raise NotImplementedError("fused communicator supports TP=1 x SP=N or TP=N x SP=1")
        self._heap = None
        self._layout = None
        self._ar_index = 0
        self._declared = False
        # True: a barrier kernel after every exchange instead of signals and in-kernel waits
        # (block-scaled fp8 linears have no wait / signal hooks); also AB200_FUSED_BARRIERS=1
        self.use_barriers = os.environ.get("AB200_FUSED_BARRIERS", "0") == "1"

    # ------------------------------------------------------------------ heap
    def setup(self, max_tokens: int, max_tp_tokens: int, blk_rows: int, hidden: int,
              attn_cols: int, swiftkv: bool = False) -> None:
        """Allocate and exchange the symmetric heap. ``max_tokens``: largest (padded) step;
        ``max_tp_tokens``: largest tensor-parallel step (also bounds the rows a step samples);
        ``attn_cols`` = SP * h * D; ``swiftkv``: the model needs the boundary buffer that
        holds the normalised hidden state of every token of a step."""
        import torch.distributed._symmetric_memory as symm_mem
        W = self.ways
        n_local = (max_tokens + self.sp - 1) // self.sp
        self._amx_rows = max(max_tp_tokens, 1)
        sizes = {
            "flags": 4096,
            "qkv": max_tokens * blk_rows * 2 if self.sp > 1 else 0,
            "attn": n_local * attn_cols * 2 if self.sp > 1 else 0,
            "ar0": max_tp_tokens * hidden * 2,
            "ar1": max_tp_tokens * hidden * 2,
            "res0": max_tp_tokens * hidden * 2,
            "res1": max_tp_tokens * hidden * 2,
            "ar2_flags": 2 * 16 * 128 * 4,
            # sampled rows handed to every rank (hidden state, residual), arg-max candidates,
            # and the SwiftKV boundary's all-token buffer
            "chan": 4 * _Channel.BYTES,
            "rows_a": max_tp_tokens * hidden * 2 if self.sp > 1 else 0,
            "rows_b": max_tp_tokens * hidden * 2 if self.sp > 1 else 0,
            "amx": 2 * W * self._amx_rows * 16,
            "x4": max_tokens * hidden * 2 if (self.sp > 1 and swiftkv) else 0,
        }
        off, layout = 0, {}
        for k, v in sizes.items():
            layout[k] = (off, v)
            off += (v + _ALIGN - 1) // _ALIGN * _ALIGN
        self._layout = layout
        self._heap = symm_mem.empty(off, dtype=torch.uint8, device=self.device)
        self._heap.zero_()
        self._hdl = symm_mem.rendezvous(self._heap, dist.group.WORLD)
        self._peer_base = [int(p) for p in self._hdl.buffer_ptrs]
        assert len(self._peer_base) == W
        self._max_tokens, self._max_tp_tokens = max_tokens, max_tp_tokens
        self._blk_rows, self._hidden, self._attn_cols = blk_rows, hidden, attn_cols
        self._flag_ptrs = _ptr_array([b + layout["flags"][0] for b in self._peer_base])
        self._epoch_ptr = self._peer_base[self.rank] + layout["flags"][0] + 1024
        self._qkv_ptrs = _ptr_array([b + layout["qkv"][0] for b in self._peer_base])
        self._ar_ptrs = [_ptr_array([b + layout[k][0] for b in self._peer_base])
                         for k in ("ar0", "ar1")]
        self._res_ptrs = [_ptr_array([b + layout[k][0] for b in self._peer_base])
                          for k in ("res0", "res1")]
        self._ar2_flag_ptrs = _ptr_array([b + layout["ar2_flags"][0] for b in self._peer_base])
        self._rows_ptrs = [_ptr_array([b + layout[k][0] for b in self._peer_base])
                           for k in ("rows_a", "rows_b")]
        self._amx_ptrs = _ptr_array([b + layout["amx"][0] for b in self._peer_base])
        self._x4_ptrs = _ptr_array([b + layout["x4"][0] for b in self._peer_base])
        cb = layout["chan"][0]
        self._chan = {name: _Channel(self._peer_base, cb + i * _Channel.BYTES, self.rank, W)
                      for i, name in enumerate(("qkv", "attn", "ar"))}
        # operand waits handed from a producing call to the call that consumes its output
        self._pending_wait = {}

        self._ar2_epochs = torch.zeros(128, dtype=torch.int32, device=self.device)
        mode = os.environ.get("AB200_ALLREDUCE", "auto").lower()
        if mode not in ("auto", "oneshot", "twoshot"):
            raise ValueError("AB200_ALLREDUCE must be auto, oneshot or twoshot")
        # Bytes of one rank's partial from which the two-shot kernel is used. Its two flag
        # exchanges and the system-scope fence between them cost about 20 us more than the
        # one-shot path (measured on two GPUs at every size); it moves (W-1)^2/W times the
        # tensor less over NVLink, so it pays once that saving is worth 20 us at ~600 GB/s:
        # 24 MB on 2 GPUs, 5.3 MB on 4, 2 MB on 8.
        auto_from = int(12e6 * W / max(1, (W - 1) ** 2)) if W > 1 else (1 << 62)
        self._two_shot_from = {"auto": auto_from, "oneshot": 1 << 62, "twoshot": 0}[mode]
        # reductions up to this many bytes per rank are folded into the following RMSNorm
        # (every rank then reads all W partials: more NVLink bytes than the two-shot kernel,
        # two launches and two flag exchanges fewer)
        self._fold_reduce_max = min(self._two_shot_from, 4 << 20)
        if os.environ.get("AB200_FOLD_REDUCE", "1") == "0":
            self._fold_reduce_max = 0
        torch.cuda.synchronize(self.device)
        dist.barrier()
        L = native.lib()
        P, I, LL, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        native.declare("ab200_barrier", I, [P, I, I, P, P, P])
        native.declare("ab200_allreduce", I, [P, I, P, P, LL, P])
        native.declare("ab200_allreduce2", I, [P, P, P, P, I, I, LL, P, P])
        native.declare("ab200_push_rows", I, [P, LL, P, LL, LL, I, I, P, P, P, LL, I, P])
        native.declare("ab200_rmsnorm_allgather", I, [P, LL, P, P, P, LL, I, I, LL, I, F, P])
        native.declare("ab200_argmax_exchange", I, [P, P, I, I, P, P, I, I, P, P, P, P, P])
        native.declare("ab200_attention_scatter_sync", I, [P, LL, P, P, LL, I, P, I, P, I, P, I, LL,
                                                           I, I, I, F, P, I, I, LL, P, P, I, P, P, P])
        native.declare("ab200_reduce_rmsnorm", I, [P, I, LL, P, P, P, LL, P, LL, P, P, LL, LL, I, F,
                                                   P, P, P])
        native.declare("ab200_linear_bf16_scatter", I, [P, LL, P, LL, P, I, I, LL, LL, I, I, I, P, P])
        native.declare("ab200_attention_scatter", I, [P, LL, P, P, LL, I, P, I, P, I, P, I, LL, I, I,
                                                      I, F, P, I, I, LL, P, P, I, P, P])
        self._lib = L

    def _view(self, key: str, rows: int, cols: int) -> torch.Tensor:
        off, size = self._layout[key]
        assert rows * cols * 2 <= size, "symmetric heap region %s too small" % key
        return self._heap[off:off + rows * cols * 2].view(torch.bfloat16).view(rows, cols)

    def device_barrier(self) -> None:
        rc = self._lib.ab200_barrier(self._flag_ptrs, self.rank, self.ways, self._epoch_ptr,
                                     native.status_buffer(self.device).data_ptr(),
                                     native.stream_ptr())
        native.check(rc, "barrier")
        ops.launch_counter.add(1)

    def begin_forward(self) -> None:
        self._ar_index = 0

    # ------------------------------------------------------- Ulysses exchanges
    def take_wait(self, name: str):
        """The operand wait that the consumer of the last ``name`` exchange must apply (once)."""
        return self._pending_wait.pop(name, None)

    def qkv_scatter_heads(self, x_local, wqkv, blk_rows: int, bias=None) -> torch.Tensor:
        """The projection's epilogue stores each head block into its owner's buffer and its last
        block signals every rank; the caller's next kernel on the result (RoPE + cache write)
        must wait with ``take_wait("qkv")``."""
        if bias is not None:
            raise NotImplementedError("a QKV bias with the fused communicator in sequence-"
                                      "parallel mode (the scattering epilogue adds none): use "
                                      "comm_backend='nccl', or tensor parallelism")
        n = x_local.shape[0]
        N = n * self.sp
        s = self.topo.sp_rank
        ch = self._chan["qkv"]
        if not isinstance(wqkv, torch.Tensor) and ops.fp8_prefers_bf16(wqkv, n):
            wqkv = ops.dequant_fp8(wqkv)          # bf16 shadow, or expanded once for long prefill
        peer = (self._qkv_ptrs, self.sp, blk_rows, s * n, blk_rows)
        from ..models.quant import Fp8RowWeight
        if isinstance(wqkv, Fp8RowWeight):
            ops.linear_fp8_row(x_local, wqkv, peer=peer,
                               sync=None if self.use_barriers else ch.sync(signal=True))
            if self.use_barriers:
                self.device_barrier()
                return self._view("qkv", N, blk_rows)
        elif not isinstance(wqkv, torch.Tensor):   # block-scaled fp8 weights: barrier kernel
            ops.linear_fp8(x_local, wqkv, peer=peer)
            self.device_barrier()
            return self._view("qkv", N, blk_rows)
        elif self.use_barriers:
            if not isinstance(x_local, torch.Tensor):
                x_local = x_local.dequantize()
            rc = ops._linear_desc(x_local.data_ptr(), x_local.stride(0), None, wqkv.data_ptr(),
                                  wqkv.stride(0), None, None, blk_rows, n, wqkv.shape[0],
                                  x_local.shape[1], None, None, None, 1, peer, None, self.device)
            native.check(rc, "linear_bf16_scatter")
            ops.launch_counter.add(1)
            self.device_barrier()
            return self._view("qkv", N, blk_rows)
        else:
            if not isinstance(x_local, torch.Tensor):
                x_local = x_local.dequantize()
            rc = ops._linear_desc(x_local.data_ptr(), x_local.stride(0), None, wqkv.data_ptr(),
                                  wqkv.stride(0), None, None, blk_rows, n, wqkv.shape[0],
                                  x_local.shape[1], None, None, None, 1, peer,
                                  ch.sync(signal=True), self.device)
            native.check(rc, "linear_bf16_scatter")
            ops.launch_counter.add(1)
        self._pending_wait["qkv"] = ch.sync(wait=True)
        return self._view("qkv", N, blk_rows)

    def attention_gather_tokens(self, q, k_cache, v_cache, meta, h, hkv, D, scale):
        N = q.shape[0]
        n = N // self.sp
        s = self.topo.sp_rank
        cols = self.sp * h * D
        off = self._layout["attn"][0] + s * h * D * 2
        ptrs = _ptr_array([b + off for b in self._peer_base])
        bt = meta.block_tables
        ch = self._chan["attn"]
        sync = ch.sync(signal=not self.use_barriers)
        rc = self._lib.ab200_attention_scatter_sync(
            q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.shape[0],
            k_cache.shape[2], bt.data_ptr(), bt.shape[1], meta.work.data_ptr(), meta.num_work,
            native.ptr(meta.tok_splits), meta.max_splits, N, h, hkv, D, float(scale), ptrs,
            self.sp, n, cols, native.ptr(meta.o_part), native.ptr(meta.lse_part), meta.tile_keys,
            ctypes.byref(sync), native.status_buffer(self.device).data_ptr(), native.stream_ptr())
        native.check(rc, "attention_scatter")
        ops.launch_counter.add(2 if meta.max_splits > 1 else 1)
        if self.use_barriers:
            self.device_barrier()
        else:
            # the o_proj (its quantiser or its load warp) waits for the ranks' signals itself
            self._pending_wait["attn"] = ch.sync(wait=True)
        return self._view("attn", n, cols)

    # ------------------------------------------------- sampled rows, SwiftKV boundary, arg-max
    def _push_rows(self, a_local, b_local, idx) -> None:
        n = a_local.shape[0]
        rc = self._lib.ab200_push_rows(
            a_local.data_ptr(), a_local.stride(0), native.ptr(b_local),
            b_local.stride(0) if b_local is not None else 0, n, self.topo.sp_rank, self.sp,
            idx.data_ptr(), self._rows_ptrs[0], self._rows_ptrs[1] if b_local is not None else None,
            idx.numel(), a_local.shape[1], native.stream_ptr())
        native.check(rc, "push_rows")
        ops.launch_counter.add(1)

    def gather_rows_all(self, h_local, res_local, idx):
        """The owner of each sampled token stores its hidden-state and residual rows into every
        rank's staging buffers (peer stores); after the barrier all ranks hold all rows."""
        B, H = idx.numel(), h_local.shape[1]
        assert res_local.stride(1) == 1 and h_local.stride(1) == 1
        self._push_rows(h_local, res_local, idx)
        self.device_barrier()
        self.stats["fused_row_gather"] = self.stats.get("fused_row_gather", 0) + 1
        return self._view("rows_a", B, H), self._view("rows_b", B, H)

    def swiftkv_boundary(self, h_local, res_local, weight, eps: float, idx):
        """The boundary norm writes its rows into every rank's all-token buffer as it produces
        them; the residual travels for the sampled rows only."""
        n, H = h_local.shape
        N = n * self.sp
        s = self.topo.sp_rank
        assert res_local.is_contiguous()
        rc = self._lib.ab200_rmsnorm_allgather(
            h_local.data_ptr(), h_local.stride(0), res_local.data_ptr(), weight.data_ptr(),
            self._x4_ptrs, s * n, s, self.sp, n, H, float(eps), native.stream_ptr())
        native.check(rc, "rmsnorm_allgather")
        ops.launch_counter.add(1)
        self._push_rows(res_local, None, idx)
        self.device_barrier()
        self.stats["fused_boundary"] = self.stats.get("fused_boundary", 0) + 1
        return self._view("x4", N, H), self._view("rows_a", idx.numel(), H)

    def argmax_exchange(self, ids: torch.Tensor, vals: torch.Tensor) -> torch.Tensor:
        """Every rank stores its (value, token) candidates into all ranks' slots, the ranks
        meet at a flag barrier inside the same kernel, and each picks the best locally."""
        B = ids.numel()
        if B > self._amx_rows:
            return super().argmax_exchange(ids, vals)
        out = torch.empty_like(ids)
        rc = self._lib.ab200_argmax_exchange(
            ids.data_ptr(), vals.data_ptr(), B, self._amx_rows, self._amx_ptrs, self._flag_ptrs,
            self.rank, self.ways, self._epoch_ptr, out.data_ptr(), None,
            native.status_buffer(self.device).data_ptr(), native.stream_ptr())
        native.check(rc, "argmax_exchange")
        ops.launch_counter.add(1)
        self.stats["fused_argmax"] = self.stats.get("fused_argmax", 0) + 1
        return out

    # --------------------------------------------------------------- reductions
    def reduce_buffer(self, rows: int, cols: int) -> torch.Tensor:
        """Heap buffer a row-parallel GEMM should write its partial product into."""
        return self._view("ar%d" % (self._ar_index & 1), rows, cols)

    def folds_reduce(self, rows: int, cols: int) -> bool:
        """Whether a [rows, cols] reduction is left to the kernel that consumes it."""
        return (not self.use_barriers and rows * cols * 2 <= self._fold_reduce_max and
                cols % 8 == 0 and cols <= 16384)

    def linear_partial(self, x, w, sync_wait=None):
        """Row-parallel linear whose partial product stays in the heap; its last block signals
        every rank. Returns the handle the consuming kernel takes."""
        rows, cols = x.shape[0], w.shape[0]
        key = self._ar_index & 1
        self._ar_index += 1
        sync = self._chan["ar"].sync(signal=True)
        if sync_wait is not None:
            sync.wait_flags, sync.wait_epoch_ctr = sync_wait.wait_flags, sync_wait.wait_epoch_ctr
            sync.wait_world = sync_wait.wait_world
        ops.linear(x, w, out=self._view("ar%d" % key, rows, cols), sync=sync)
        return PendingReduce(key, rows, cols)

    def reduce_rmsnorm(self, pend: PendingReduce, weight, eps: float, residual=None,
                       quant: bool = False):
        """sum over ranks -> (+ residual, in place) -> RMSNorm -> bf16 rows or a ``QuantAct``."""
        rows, cols = pend.rows, pend.cols
        dev = self.device
        y = yq = sy = None
        if quant:
            from ..models.quant import QuantAct
            yq = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=dev)
            sy = torch.empty(rows, dtype=torch.float32, device=dev)
        else:
            y = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        if residual is not None:
            assert residual.is_contiguous()
        sync = self._chan["ar"].sync(wait=True)
        rc = self._lib.ab200_reduce_rmsnorm(
            self._ar_ptrs[pend.key], self.ways, cols, native.ptr(residual), weight.data_ptr(),
            native.ptr(y), cols, native.ptr(yq), cols, native.ptr(sy), None, 0, rows, cols,
            float(eps), ctypes.byref(sync), native.status_buffer(dev).data_ptr(),
            native.stream_ptr())
        native.check(rc, "reduce_rmsnorm")
        ops.launch_counter.add(1)
        self.stats["fused_reduce_norm"] = self.stats.get("fused_reduce_norm", 0) + 1
        return QuantAct(yq, sy) if quant else y

    def realize(self, pend: PendingReduce) -> torch.Tensor:
        """The reduced rows of a pending product as a plain tensor."""
        rows, cols = pend.rows, pend.cols
        out = torch.empty(rows, cols, dtype=torch.bfloat16, device=self.device)
        sync = self._chan["ar"].sync(wait=True)
        rc = self._lib.ab200_reduce_rmsnorm(
            self._ar_ptrs[pend.key], self.ways, cols, None, None, None, 0, None, 0, None,
            out.data_ptr(), cols, rows, cols, 0.0, ctypes.byref(sync),
            native.status_buffer(self.device).data_ptr(), native.stream_ptr())
        native.check(rc, "reduce_rows")
        ops.launch_counter.add(1)
        return out

    def all_reduce_full(self, t: torch.Tensor) -> torch.Tensor:
        rows, cols = t.shape
        key = self._ar_index & 1
        buf = self._view("ar%d" % key, rows, cols)
        if t.data_ptr() != buf.data_ptr():
            buf.copy_(t)
        self._ar_index += 1
        if rows * cols * 2 >= self._two_shot_from and (rows * cols) % 8 == 0:
            rc = self._lib.ab200_allreduce2(
                self._ar_ptrs[key], self._res_ptrs[key], self._ar2_flag_ptrs,
                self._ar2_epochs.data_ptr(), self.rank, self.ways, rows * cols,
                native.status_buffer(self.device).data_ptr(), native.stream_ptr())
            native.check(rc, "allreduce2")
            ops.launch_counter.add(1)
            # valid until the second reduction after this one reuses the buffer
            return self._view("res%d" % key, rows, cols)
        self.device_barrier()
        out = torch.empty(rows, cols, dtype=t.dtype, device=t.device)
        rc = self._lib.ab200_allreduce(self._ar_ptrs[key], self.ways, out.data_ptr(), None,
                                       rows * cols, native.stream_ptr())
        native.check(rc, "allreduce")
        ops.launch_counter.add(1)
        return out

    def all_reduce_tp(self, t: torch.Tensor) -> torch.Tensor:
        # TP=N x SP=1: the TP group is the whole grid
        return self.all_reduce_full(t)
