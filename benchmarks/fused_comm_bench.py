"""Fused compute+collective kernels against their "GEMM, then NCCL" equivalents, on N GPUs
of one node (one process per GPU):

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/fused_comm_bench.py

Cases (Llama-3.1-8B shapes, bf16; n = tokens per rank):

* qkv_scatter: QKV projection whose epilogue stores every head shard into the rank that owns
  it (Ulysses sequence -> head exchange) and signals from its last block, followed by a
  consumer kernel (the activation quantiser over the received rows) that waits for the ranks'
  signals, vs the same GEMM into local memory, ``all_to_all_single`` and the same consumer;
* attention_scatter: attention over all ranks' tokens for this rank's heads whose epilogue
  stores every token's output row into the rank that owns the token (Ulysses head -> sequence
  exchange), followed by the consumer that waits, vs attention into local memory,
  ``all_to_all_single``, the re-layout copy and the same consumer (prefill: sequences of up to
  2048 tokens; at 64 tokens per rank: one query token per sequence over 2000 cached tokens);
* gemm_reduce_norm: row-parallel o_proj leaving its partial product in the symmetric heap +
  the kernel that waits for the ranks' signals, sums the partials, adds the residual and
  normalises, vs the GEMM, ``dist.all_reduce`` and the RMSNorm(+residual) kernel;
* allreduce: row-parallel o_proj writing its partial product into the symmetric heap + the
  peer-memory all-reduce (one-shot and two-shot kernels) vs the GEMM + ``dist.all_reduce``.

Times are CUDA events on the launching stream, median of ``--iters`` after warm-up, maximum
over ranks. For each fused case the roofline time is the slower of FLOPs / measured bf16 peak
and bytes sent per GPU / 770 GB/s (measured peer-copy bandwidth per direction on this pool;
nominal 900), for attention also its K/V bytes / 6533.5 GB/s measured copy bandwidth; the
printed fraction is roofline time / measured time.
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from arcticinference_b200 import ops  # noqa: E402
from arcticinference_b200.parallel.comm import init_communicator  # noqa: E402

LINK_GBS = 770.0
HBM_GBS = 6533.5     # measured copy bandwidth of this pool (decode attention is bound by KV bytes)


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)).get("bf16_tflops", 1590.0)
    return 1590.0


def timed(fn, iters, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(200000)          # let the host queue ahead of the device
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t) * 1e3                   # microseconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", default="4096,512,64", help="tokens per rank, comma list")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    comm = init_communicator(1, world, backend="fused")
    rank, dev = comm.rank, comm.device
    H, Hq, Hkv, D = 4096, 32, 8, 128
    h, hkv = Hq // world, max(1, Hkv // world)
    blk = (h + 2 * hkv) * D
    sizes = [int(t) for t in a.tokens.split(",")]
    nmax = max(sizes)
    comm.setup(nmax * world, nmax * world, blk, H, world * h * D)
    peak = peaks()
    R = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
    wqkv = R(world * blk, H)               # rank-major head blocks
    wo = R(H, h * D)                       # this rank's o_proj columns
    res = []
    for n in sizes:
        x = R(n, H)
        # ---- QKV GEMM with the head exchange in its epilogue
        def fused_x1():
            view = comm.qkv_scatter_heads(x, wqkv, blk)
            return ops.quant_fp8_row(view, sync=comm.take_wait("qkv"))

        t_fused = timed(fused_x1, a.iters)
        send = torch.empty(n, world * blk, dtype=torch.bfloat16, device=dev)
        recv = torch.empty(world * n, blk, dtype=torch.bfloat16, device=dev)

        def unfused():
            ops.linear(x, wqkv, out=send)
            # [n, W*blk] -> W chunks of [n, blk]
            chunks = send.view(n, world, blk).transpose(0, 1).contiguous()
            dist.all_to_all_single(recv.view(world, n, blk), chunks)
            return ops.quant_fp8_row(recv)

        t_base = timed(unfused, a.iters)
        flops = 2.0 * n * world * blk * H
        sent = n * (world - 1) * blk * 2.0
        roof = max(flops / (peak * 1e12), sent / (LINK_GBS * 1e9)) * 1e6
        res.append({"case": "qkv_scatter", "tokens_per_rank": n, "fused_us": t_fused, "gemm_then_nccl_us": t_base,
                    "speedup": t_base / t_fused, "roofline_us": roof, "fraction_of_roofline": roof / t_fused,
                    "bytes_sent_per_gpu": sent, "flops": flops})
        # ---- attention with the head -> sequence exchange in its epilogue
        N = n * world
        if n >= 256:
            seq = min(N, 2048)
            q_lens = [seq] * (N // seq)
            kv_lens = list(q_lens)
        else:
            q_lens, kv_lens = [1] * N, [2000] * N
        bs = 64
        nblk = [(k + bs - 1) // bs for k in kv_lens]
        bt = torch.zeros(len(q_lens), max(nblk), dtype=torch.int32)
        o = 1
        for i, nb in enumerate(nblk):
            bt[i, :nb] = torch.arange(o, o + nb)
            o += nb
        q_in, kc, vc = R(N, h * D), R(o, hkv, bs, D), R(o, hkv, bs, D)
        meta = ops.build_attention_metadata(q_lens, kv_lens, bt.to(dev), h // hkv, h, D, dev, Hkv=hkv)
        scale = D ** -0.5

        def fused_x2():
            view = comm.attention_gather_tokens(q_in, kc, vc, meta, h, hkv, D, scale)
            return ops.quant_fp8_row(view, sync=comm.take_wait("attn"))

        recv2 = torch.empty(world, n, h * D, dtype=torch.bfloat16, device=dev)

        def unfused_x2():
            out = ops.attention(q_in, kc, vc, meta, h, hkv, D, scale)
            dist.all_to_all_single(recv2, out.view(world, n, h * D))
            return ops.quant_fp8_row(recv2.transpose(0, 1).reshape(n, world * h * D))

        t_f, t_b = timed(fused_x2, a.iters), timed(unfused_x2, a.iters)
        flops = sum(4.0 * a_ * (b_ - a_ / 2.0) * h * D for a_, b_ in zip(q_lens, kv_lens))
        sent = n * (world - 1) * h * D * 2.0
        kv_bytes = sum(kv_lens) * hkv * D * 2 * 2.0       # K and V of this rank's heads, read once
        roof = max(flops / (peak * 1e12), sent / (LINK_GBS * 1e9), kv_bytes / (HBM_GBS * 1e9)) * 1e6
        res.append({"case": "attention_scatter", "tokens_per_rank": n, "fused_us": t_f,
                    "attention_then_nccl_us": t_b, "speedup": t_b / t_f, "roofline_us": roof,
                    "fraction_of_roofline": roof / t_f, "bytes_sent_per_gpu": sent, "flops": flops})
        del kc, vc, q_in
        # ---- row-parallel GEMM + all-reduce
        a_in = R(n, h * D)

        def fused_ar():
            comm.begin_forward()
            buf = comm.reduce_buffer(n, H)
            ops.linear(a_in, wo, out=buf)
            return comm.all_reduce_full(buf)

        out_local = torch.empty(n, H, dtype=torch.bfloat16, device=dev)

        def nccl_ar():
            ops.linear(a_in, wo, out=out_local)
            dist.all_reduce(out_local)

        t_b = timed(nccl_ar, a.iters)
        flops = 2.0 * n * H * h * D
        for algo, from_bytes in (("one_shot", 1 << 62), ("two_shot", 0)):
            comm._two_shot_from = from_bytes
            t_f = timed(fused_ar, a.iters)
            # bytes one rank pulls over NVLink: one-shot reads every other rank's partial in
            # full; two-shot reads (W-1)/W of the tensor and writes as much the other way
            moved = n * H * 2.0 * ((world - 1) if algo == "one_shot" else (world - 1) / world)
            roof = max(flops / (peak * 1e12), moved / (LINK_GBS * 1e9)) * 1e6
            res.append({"case": "gemm_allreduce_" + algo, "tokens": n, "fused_us": t_f,
                        "gemm_then_nccl_us": t_b, "speedup": t_b / t_f, "roofline_us": roof,
                        "fraction_of_roofline": roof / t_f, "bytes_read_per_gpu": moved,
                        "flops": flops})
        # ---- row-parallel GEMM + reduction folded into the following RMSNorm
        if comm.folds_reduce(n, H):
            gamma = R(H)
            resid = R(n, H)

            def fused_rn():
                comm.begin_forward()
                pend = comm.linear_partial(a_in, wo)
                return comm.reduce_rmsnorm(pend, gamma, 1e-5, residual=resid)

            def nccl_rn():
                ops.linear(a_in, wo, out=out_local)
                dist.all_reduce(out_local)
                return ops.rmsnorm(out_local, gamma, 1e-5, residual=resid)

            t_f, t_b2 = timed(fused_rn, a.iters), timed(nccl_rn, a.iters)
            moved = n * H * 2.0 * (world - 1)
            roof = max(flops / (peak * 1e12), moved / (LINK_GBS * 1e9)) * 1e6
            res.append({"case": "gemm_reduce_norm", "tokens": n, "fused_us": t_f,
                        "gemm_nccl_norm_us": t_b2, "speedup": t_b2 / t_f, "roofline_us": roof,
                        "fraction_of_roofline": roof / t_f, "bytes_read_per_gpu": moved,
                        "flops": flops})
    ops.check_status()
    if rank == 0:
        for r in res:
            print(json.dumps(r))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
