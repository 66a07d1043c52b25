"""Micro-benchmarks of the hot kernels, one case per invocation (also the workload for
``ncu`` captures: each case launches its kernel a handful of times on inputs larger than
L2 but of at most a few GB).

    python benchmarks/kernel_bench.py --case gemm_prefill   [--iters 20]
    python benchmarks/kernel_bench.py --case attn_decode --no-time   # for ncu: 3 launches only

Timing: CUDA events around each launch, median reported, with achieved TFLOP/s or GB/s
against the measured peaks in MEASURED_PEAKS.json when present. Before the first event of an
iteration the stream is given ~200 us of busy-waiting to chew on, so that the host has queued
the event pair and the launch by the time the device reaches them: the interval is then the
device's own time for the kernel, not the host's launch path (which for a 10 us decode kernel
would otherwise be most of the number). Every case keeps several
copies of its large operand (weights, KV cache, activations) whose total exceeds twice the
L2 capacity and rotates through them, so each timed launch reads its operands from HBM
without the write-back traffic that a dirty flush buffer would add to the measurement.
"""

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200 import ops  # noqa: E402

DEV = "cuda:0"


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def R(*s):
    return (torch.randn(*s, device=DEV) * 0.05).to(torch.bfloat16)


ROTATE_BYTES = 320 << 20      # > 2 x the 126 MB L2


def copies_for(nbytes: int) -> int:
    return max(1, min(64, -(-ROTATE_BYTES // max(int(nbytes), 1))))


def timeit(fn, iters, warm=3, copies=1):
    """``fn(i)`` launches the case on operand copy ``i % copies`` (``fn()`` when copies == 1:
    such a case must stream more than L2 by itself)."""
    call = (lambda i: fn()) if copies == 1 else (lambda i: fn(i % copies))
    for i in range(max(warm, copies)):
        call(i)
    torch.cuda.synchronize()
    ts = []
    for i in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(400000)     # head start for the host (~200 us of device time)
        e0.record()
        call(i)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def paged(q_lens, kv_lens, Hq=32, Hkv=8, D=128, bs=64):
    T = sum(q_lens)
    nblk = [(k + bs - 1) // bs for k in kv_lens]
    bt = torch.zeros(len(q_lens), max(nblk), dtype=torch.int32)
    o = 1
    for i, n in enumerate(nblk):
        bt[i, :n] = torch.arange(o, o + n)
        o += n
    q, kc, vc = R(T, Hq * D), R(o, Hkv, bs, D), R(o, Hkv, bs, D)
    meta = ops.build_attention_metadata(q_lens, kv_lens, bt.to(DEV), Hq // Hkv, Hq, D, DEV)
    return q, kc, vc, meta


CASES = {
    # name: (kind, params)
    "gemm_prefill": ("gemm", (8192, 28672, 4096)),
    "gemm_prefill_qkv": ("gemm", (8192, 6144, 4096)),
    "gemm_prefill_down": ("gemm", (8192, 4096, 14336)),
    "gemm_decode": ("gemm", (32, 28672, 4096)),
    "gemm_decode_128": ("gemm", (128, 28672, 4096)),
    "gemm_decode_128_down": ("gemm", (128, 4096, 14336)),
    "gemm_decode_o": ("gemm", (32, 4096, 4096)),
    "gemm_decode_down": ("gemm", (32, 4096, 14336)),
    "gemm_mid": ("gemm", (512, 28672, 4096)),
    "gemm_fp8_prefill": ("gemm_fp8", (8192, 28672, 4096)),
    "gemm_fp8_mid": ("gemm_fp8", (256, 28672, 4096)),
    "gemm_fp8_decode": ("gemm_fp8", (32, 28672, 4096)),
    "gemm_fp8_decode_128": ("gemm_fp8", (128, 28672, 4096)),
    "gemm_fp8_decode_o": ("gemm_fp8", (32, 4096, 4096)),
    "gemm_fp8_decode_down": ("gemm_fp8", (32, 4096, 14336)),
    # W8A8 with per-token / per-feature scales (activations already quantised, as the fused
    # norm / SiLU kernels hand them over); "*_w8a8_block" is the block-scaled kernel itself
    "gemm_fp8row_prefill": ("gemm_fp8row", (8192, 28672, 4096)),
    "gemm_fp8row_prefill_qkv": ("gemm_fp8row", (8192, 6144, 4096)),
    "gemm_fp8row_prefill_down": ("gemm_fp8row", (8192, 4096, 14336)),
    "gemm_fp8row_mid": ("gemm_fp8row", (512, 28672, 4096)),
    "gemm_fp8row_decode": ("gemm_fp8row", (32, 28672, 4096)),
    "gemm_fp8row_decode_128": ("gemm_fp8row", (128, 28672, 4096)),
    "gemm_fp8row_decode_128_down": ("gemm_fp8row", (128, 4096, 14336)),
    "gemm_fp8row_decode_o": ("gemm_fp8row", (32, 4096, 4096)),
    "gemm_fp8row_decode_128_tiled": ("gemm_fp8row_tiled", (128, 28672, 4096)),
    "gemm_fp8row_decode_128_down_tiled": ("gemm_fp8row_tiled", (128, 4096, 14336)),
    "gemm_fp8row_prefill_tiled": ("gemm_fp8row_tiled", (8192, 28672, 4096)),
    "gemm_fp8row_decode_qkv": ("gemm_fp8row", (128, 6144, 4096)),
    "gemm_w8a8_block_prefill": ("gemm_fp8blk", (8192, 28672, 4096)),
    "attn_prefill": ("attn", ([8192], [8192])),
    "attn_prefill_4x2048": ("attn", ([2048] * 4, [2048] * 4)),
    "attn_decode": ("attn", ([1] * 32, [2000] * 32)),
    "attn_decode_128": ("attn", ([1] * 128, [2000] * 128)),
    "attn_decode_long": ("attn", ([1] * 8, [8000] * 8)),
    "attn_verify": ("attn", ([4] * 32, [2000] * 32)),
    "rmsnorm": ("rmsnorm", (8192, 4096)),
    "rmsnorm_quant": ("rmsnorm_q", (8192, 4096)),
    "silu_mul": ("silu", (8192, 14336)),
    "silu_mul_quant": ("silu_q", (8192, 14336)),
    "quant_fp8_row": ("quant_row", (8192, 4096)),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True,
                    help="one of: %s (or several, comma-separated; 'all' for every case)"
                         % ", ".join(sorted(CASES)))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-time", action="store_true", help="three plain launches (for ncu)")
    ap.add_argument("--splits", type=int, default=0,
                    help="force the split-K factor of the bf16 GEMM cases (0 = the kernel's choice)")
    ap.add_argument("--tile-keys", type=int, default=0,
                    help="force the key-tile size (64 or 128) of the attention cases")
    a = ap.parse_args()
    names = sorted(CASES) if a.case == "all" else a.case.split(",")
    for name in names:
        if name not in CASES:
            raise SystemExit("unknown case %r" % name)
        run_case(a, name)
        torch.cuda.empty_cache()


def run_case(a, case):
    hbm, tf, src = peaks()
    kind, prm = CASES[case]
    if kind == "gemm":
        M, N, K = prm
        nc = copies_for(2 * N * K)
        x, ws = R(M, K), [R(N, K) for _ in range(nc)]
        fn = lambda i=0: ops.linear(x, ws[i], force_splits=a.splits)
        flops, byts = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
    elif kind == "gemm_fp8":
        from arcticinference_b200.models import quant
        M, N, K = prm
        nc = copies_for(N * K)
        x, ws = R(M, K), [quant.quantize_weight_fp8(R(N, K)) for _ in range(nc)]
        fn = lambda i=0: ops.linear(x, ws[i])
        flops, byts = 2.0 * M * N * K, 2.0 * (M * K + M * N) + 1.0 * N * K
    elif kind in ("gemm_fp8row", "gemm_fp8row_tiled"):
        from arcticinference_b200.models import quant
        M, N, K = prm
        nc = copies_for(N * K)
        xq = ops.quant_fp8_row(R(M, K))
        tiled = kind != "gemm_fp8row"     # the "_tiled" cases store 16-row x 128-byte tiles
        ws = [quant.quantize_weight_fp8_row(R(N, K), tiled=tiled) for _ in range(nc)]
        for w_ in ws:
            ops.mark_static(w_)      # parameters, as in a loaded model
        fn = lambda i=0: ops.linear(xq, ws[i], force_splits=a.splits)
        flops, byts = 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N
    elif kind == "gemm_fp8blk":
        from arcticinference_b200.models import quant
        M, N, K = prm
        nc = copies_for(N * K)
        x, ws = R(M, K), [quant.quantize_weight_fp8(R(N, K)) for _ in range(nc)]
        fn = lambda i=0: ops.linear_fp8(x, ws[i], mode="w8a8")
        flops, byts = 2.0 * M * N * K, 2.0 * (M * K + M * N) + 1.0 * N * K
    elif kind == "attn":
        ql, kl = prm
        byts = sum(b_ * 8 * 128 * 2 * 2.0 for b_ in kl) + 2.0 * sum(ql) * 32 * 128 * 2
        nc = copies_for(byts)
        sets = [paged(ql, kl) for _ in range(nc)]
        if a.tile_keys:
            for st in sets:
                st[3].tile_keys = a.tile_keys
        fn = lambda i=0: ops.attention(sets[i][0], sets[i][1], sets[i][2], sets[i][3], 32, 8, 128)
        flops = sum(4.0 * a_ * (b_ - a_ / 2.0) * 32 * 128 for a_, b_ in zip(ql, kl))
    elif kind == "rmsnorm":
        T, H = prm
        nc = copies_for(4 * T * H)
        xs, w, rs = [R(T, H) for _ in range(nc)], R(H), [R(T, H) for _ in range(nc)]
        fn = lambda i=0: ops.rmsnorm(xs[i], w, 1e-5, residual=rs[i])
        flops, byts = 0.0, 4.0 * T * H * 2
    elif kind == "rmsnorm_q":
        T, H = prm
        nc = copies_for(4 * T * H)
        xs, w, rs = [R(T, H) for _ in range(nc)], R(H), [R(T, H) for _ in range(nc)]
        fn = lambda i=0: ops.rmsnorm(xs[i], w, 1e-5, residual=rs[i], quant=True)
        flops, byts = 0.0, 3.0 * T * H * 2 + T * H
    elif kind == "quant_row":
        T, H = prm
        nc = copies_for(2 * T * H)
        xs = [R(T, H) for _ in range(nc)]
        fn = lambda i=0: ops.quant_fp8_row(xs[i])
        flops, byts = 0.0, 3.0 * T * H
    elif kind == "silu_q":
        T, I = prm
        nc = copies_for(4 * T * I)
        gs = [R(T, 2 * I) for _ in range(nc)]
        fn = lambda i=0: ops.silu_mul_blocked(gs[i], 1, quant=True)
        flops, byts = 0.0, 2.0 * T * I * 2 + T * I
    else:
        T, I = prm
        nc = copies_for(4 * T * I)
        gs = [R(T, 2 * I) for _ in range(nc)]
        fn = lambda i=0: ops.silu_mul(gs[i])
        flops, byts = 0.0, 3.0 * T * I * 2
    if a.no_time:
        for i in range(3):
            fn(i % nc)
        torch.cuda.synchronize()
        ops.check_status()
        print("ran", case)
        return
    ms = timeit(fn, a.iters, copies=nc)
    ops.check_status()
    t = ms / 1e3
    print(json.dumps({"case": case, "splits": a.splits, "us": ms * 1e3, "tflops": flops / t / 1e12,
                      "gbs": byts / t / 1e9, "frac_of_%s_bf16" % src: flops / t / 1e12 / tf,
                      "frac_of_%s_hbm" % src: byts / t / 1e9 / hbm}))


if __name__ == "__main__":
    main()
