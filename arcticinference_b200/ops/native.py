"""ctypes bridge to ``_kernels.so`` (the sm_100a kernel library, ``csrc/api.h``).

Every wrapper launches on the current torch CUDA stream and raises when the
library rejects an argument or a launch fails. Kernels never trap: bounded
waits and index checks report through a per-device int32[8] status buffer that
:func:`check_status` turns into a Python exception.
"""

from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_longlong, c_size_t, c_float

import torch

from .. import build as _build

_lib = None
_status: dict[int, torch.Tensor] = {}
_workspace: dict[int, torch.Tensor] = {}

WORKSPACE_BYTES = 96 << 20


class PeerSync(ctypes.Structure):
    """``Ab200PeerSync`` (csrc/api.h): completion signal / operand wait of one kernel launch."""
    _fields_ = [("sig_flag_ptrs", c_void_p), ("sig_done_ctr", c_void_p),
                ("sig_epoch_ctr", c_void_p), ("sig_rank", c_int), ("sig_world", c_int),
                ("wait_flags", c_void_p), ("wait_epoch_ctr", c_void_p), ("wait_world", c_int)]


class LinearDesc(ctypes.Structure):
    """``Ab200LinearDesc`` (csrc/api.h)."""
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("sx", c_void_p),
                ("w", c_void_p), ("ldw", c_longlong), ("sw", c_void_p),
                ("out", c_void_p), ("ldo", c_longlong),
                ("M", c_int), ("N", c_int), ("K", c_int),
                ("bias", c_void_p), ("residual", c_void_p), ("ldr", c_longlong), ("act", c_int),
                ("workspace", c_void_p), ("workspace_bytes", c_size_t), ("force_splits", c_int),
                ("peer_ptrs", c_void_p), ("world", c_int), ("peer_cols", c_int),
                ("peer_row_off", c_longlong),
                ("sync", PeerSync), ("status", c_void_p),
                ("w_tile_stride_n", c_longlong), ("w_tile_stride_k", c_longlong),
                ("w_static", c_int)]


class KernelError(RuntimeError):
    pass


class KernelTimeout(KernelError):
    """A bounded device-side wait ran out (barrier or peer flag)."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _build.load_kernels()
        _declare(_lib)
    return _lib


def _declare(L: ctypes.CDLL) -> None:
    P, I, LL, F, SZ = c_void_p, c_int, c_longlong, c_float, c_size_t
    sigs = {
        "ab200_linear_bf16_workspace_bytes": (SZ, [I, I, I]),
        "ab200_linear_bf16": (I, [P, LL, P, LL, P, LL, I, I, I, P, P, LL, I, P, SZ, I, P, P]),
        "ab200_gemm_bf16_nn": (I, [P, LL, P, LL, P, LL, I, I, I, P, P]),
        "ab200_embedding": (I, [P, P, P, LL, I, LL, LL, P]),
        "ab200_rmsnorm": (I, [P, LL, P, P, P, LL, LL, I, F, P]),
        "ab200_layernorm": (I, [P, P, P, P, P, LL, I, F, P]),
        "ab200_silu_mul": (I, [P, P, LL, I, I, P]),
        "ab200_rope_cache": (I, [P, LL, P, P, P, P, P, LL, I, I, I, I, LL, I, P, P]),
        "ab200_gather_rows": (I, [P, LL, P, P, LL, I, P]),
        "ab200_bert_embed_ln": (I, [P, P, P, P, P, P, P, P, P, LL, I, LL, LL, LL, F, P, P]),
        "ab200_pool_normalize": (I, [P, LL, P, P, I, I, I, I, P]),
        "ab200_kv_bulk_write": (I, [P, LL, P, P, P, P, P, P, P, LL, I, I, I, I, LL, I, P, P]),
        "ab200_kv_write_fp4": (I, [P, LL, P, LL, P, P, P, P, P, LL, I, I, I, LL, P, P]),
        "ab200_kv_read_fp4": (I, [P, P, P, P, LL, LL, I, I, I, P]),
        "ab200_patch_ids": (I, [P, P, P, LL, LL, P]),
        "ab200_argmax_sample": (I, [P, I, LL, LL, I, P, P, P, P, LL, P]),
        "ab200_quant_fp8": (I, [P, LL, P, LL, P, LL, LL, I, P]),
        "ab200_dequant_fp8": (I, [P, LL, P, LL, P, LL, LL, I, P]),
        "ab200_linear_w8a16": (I, [P, LL, P, LL, P, LL, P, LL, I, I, I, P, SZ, I, P, I, I, LL, P, P]),
        "ab200_linear_fp8": (I, [P, LL, P, LL, P, LL, P, LL, P, LL, I, I, I, P, SZ, I, P, I, I, LL,
                                 P, P]),
        "ab200_linear_fp8_row": (I, [P, LL, P, P, LL, P, P, LL, I, I, I, P, P, LL, I, P, SZ, I, P,
                                     I, I, LL, P, P]),
        "ab200_quant_fp8_row": (I, [P, LL, P, LL, P, LL, I, P]),
        "ab200_rmsnorm_quant": (I, [P, LL, P, P, P, LL, P, P, LL, LL, I, F, P]),
        "ab200_silu_mul_quant": (I, [P, P, LL, P, LL, I, I, P]),
        "ab200_linear_desc": (I, [P, P]),
        "ab200_rope_cache_wait": (I, [P, LL, P, P, P, P, P, LL, I, I, I, I, LL, I, P, P, P]),
        "ab200_topk_topp_mask": (I, [P, LL, P, LL, I, I, P, P, P, P]),
        "ab200_qk_norm": (I, [P, LL, P, P, LL, I, I, I, F, P, P, P]),
        "ab200_quant_fp8_row_wait": (I, [P, LL, P, LL, P, LL, I, P, P, P]),
        "ab200_spec_ln": (I, [P, LL, P, P, P, LL, LL, I, F, F, P]),
        "ab200_mlp_spec_step": (I, [P, LL, P, P, F, P, P, P, LL, LL, I, F, I, P]),
        "ab200_sum_lstm": (I, [P, LL, P, I, P, F, P, LL, P, P, P, P, P, P, LL, LL, I, F, I, P]),
        "ab200_verify_greedy": (I, [P, P, P, P, I, I, P, P, P, P, P]),
        "ab200_attention": (I, [P, LL, P, P, LL, LL, I, P, I, P, I, P, I, LL, I, I, I, I, F, P,
                                LL, P, P, P, I, P, P]),
    }
    for name, (res, args) in sigs.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args


def declare(name: str, restype, argtypes) -> None:
    """Register the signature of an entry point added by another module."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status_buffer(device: torch.device | int | None = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    buf = _status.get(idx)
    if buf is None:
        buf = torch.zeros(8, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = buf
    return buf


def workspace(device: torch.device | int | None = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    buf = _workspace.get(idx)
    if buf is None:
        buf = torch.empty(WORKSPACE_BYTES, dtype=torch.uint8, device=f"cuda:{idx}")
        _workspace[idx] = buf
    return buf


_CODES = {1: "mbarrier wait timed out", 2: "peer flag wait timed out",
          3: "index check failed", 4: "bad argument"}


_timeouts = 0


def timeout_count() -> int:
    """How many times ``check_status`` has found a device-side wait that ran out."""
    return _timeouts


def check_status(device=None, reset: bool = True) -> None:
    """Synchronise and raise if any kernel on ``device`` recorded an error."""
    buf = status_buffer(device)
    vals = buf.tolist()  # synchronises
    if vals[0] != 0:
        if reset:
            buf.zero_()
        msg = "%s (code %d, block %d, detail %d/%d)" % (
            _CODES.get(vals[0], "unknown"), vals[0], vals[1], vals[2], vals[3])
        if vals[0] in (1, 2):
            global _timeouts
            _timeouts += 1
            raise KernelTimeout(msg)
        raise KernelError(msg)


def check(rc: int, what: str) -> None:
    if rc != 0:
        reasons = {-2: "unsupported shape/alignment", -3: "cudaFuncSetAttribute failed",
                   -4: "tensor map creation failed", -5: "kernel launch failed",
                   -6: "size exceeds the built-in limit"}
        raise KernelError("%s: %s (rc=%d)" % (what, reasons.get(rc, "error"), rc))
