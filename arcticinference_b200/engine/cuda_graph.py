"""CUDA-graph replay of decode-shaped steps.

A step is decode-shaped when every scheduled request feeds only its last token
plus its draft tokens (no prompt chunk), so every row is sampled. Such steps are
launch-bound (about ten kernels per layer), so the whole forward pass + LM head +
arg-max is captured once per (mode, padded token count) and replayed.

Static shapes: token count padded to a bucket; block table ``[bucket,
max_blocks_per_seq]``; attention work list ``[bucket * splits, 8]`` whose unused
entries are no-ops; split-KV scratch sized for ``splits``. Per step only the
contents of those buffers change (two pinned-to-device copies).

Bucket tables follow the reference's dual tables
(arctic_inference/vllm/ulysses.py:544-618): tensor-parallel (shift) steps use the
canonical sizes 1, 2, 4, 8, 16, ... step 8 to 256, step 16 to 512; sequence-parallel
steps use those sizes times SP so that the per-rank shapes stay canonical.
"""

from __future__ import annotations

import torch

from .. import ops
from ..models.llama import ForwardBatch


def canonical_sizes(limit: int = 512) -> list[int]:
    s = [1, 2, 4] + list(range(8, 257, 8)) + list(range(272, 513, 16))
    return [x for x in s if x <= limit]


def bucket_for(n: int, sizes: list[int]):
    for s in sizes:
        if s >= n:
            return s
    return None


class DecodeGraph:
    def __init__(self, runner, mode: str, bucket: int):
        self.runner = runner
        self.mode = mode
        self.bucket = bucket
        m = runner.model
        dev = runner.device
        cfg = runner.config
        self.max_blocks = (cfg.scheduler.max_model_len + runner.block_size - 1) // runner.block_size
        hkv = m.hkv
        # enough KV splits to occupy the GPU when the batch is small; for a large batch the
        # sequences of the last, partly filled wave of CTAs are cut (ops.tail_split_plan)
        max_q = 1 + (cfg.speculative.max_draft_tokens if cfg.speculative else 0)
        small_tiles = max_q * runner.G <= 32 and runner.block_size <= 64
        self.splits = int(max(1, min(16, 148 // max(1, bucket * hkv))))
        self.work_cap = bucket * self.splits + 1
        n_cut, pieces = ops.tail_split_plan(bucket, hkv, 148 * (2 if small_tiles else 1))
        if self.splits == 1 and n_cut > 0 and max_q == 1:
            self.splits = pieces
            self.work_cap = bucket + n_cut * (pieces - 1) + 1
        n64 = 4 * bucket      # ids | positions | slots | source rows of run-ahead tokens
        n32 = bucket * self.max_blocks + self.work_cap * 8 + bucket
        pin = dev.type == "cuda"
        self.h64 = torch.zeros(n64, dtype=torch.int64, pin_memory=pin)
        self.h32 = torch.zeros(n32, dtype=torch.int32, pin_memory=pin)
        self.d64 = torch.zeros(n64, dtype=torch.int64, device=dev)
        self.d32 = torch.zeros(n32, dtype=torch.int32, device=dev)
        B, MB = bucket, self.max_blocks
        self.meta = ops.AttentionMetadata([], [], bucket)
        self.meta.block_tables = self.d32[:B * MB].view(B, MB)
        self.meta.work = self.d32[B * MB:B * MB + self.work_cap * 8].view(self.work_cap, 8)
        self.meta.tok_splits = self.d32[B * MB + self.work_cap * 8:]
        self.meta.num_work = self.work_cap
        self.meta.max_splits = self.splits
        self.meta.tile_keys = 64 if small_tiles else 128
        if self.splits > 1:
            self.meta.o_part = torch.empty(self.splits, B, m.h, m.D, dtype=torch.float32, device=dev)
            self.meta.lse_part = torch.empty(self.splits, B, m.h, dtype=torch.float32, device=dev)
        self.logits_indices = torch.arange(bucket, dtype=torch.int64, device=dev)
        self.batch = ForwardBatch(input_ids=self.d64[:B], positions=self.d64[B:2 * B],
                                  slots=self.d64[2 * B:3 * B], attn_meta=self.meta,
                                  logits_indices=self.logits_indices, num_tokens=B, mode=mode)
        if cfg.model.is_swiftkv:
            self.batch.sel_positions = self.batch.positions
            self.batch.sel_attn_meta = self.meta
        self.graph = None
        self.ids_out = None
        self.hidden_out = None
        self.launches = 0
        self._uploaded = torch.cuda.Event() if pin else None
        self._upload_pending = False

    # ------------------------------------------------------------- host staging
    def wait_uploaded(self) -> None:
        """The pinned buffers may be rewritten once the previous upload has left them."""
        if self._upload_pending and self._uploaded is not None:
            self._uploaded.synchronize()
            self._upload_pending = False

    def fill(self, out, src_rows=None) -> list:
        """Write this step's inputs into the pinned buffers. Returns rows per request.
        ``src_rows[t]`` >= 0: token t is the previous step's sampled token at that row."""
        r = self.runner
        bs = r.block_size
        B, MB = self.bucket, self.max_blocks
        h64 = self.h64.numpy()
        h32 = self.h32.numpy()
        ids, pos, slots = h64[:B], h64[B:2 * B], h64[2 * B:3 * B]
        src = h64[3 * B:4 * B]
        src[:] = -1
        if src_rows is not None:
            src[:len(src_rows)] = src_rows
        bt = h32[:B * MB].reshape(B, MB)
        work = h32[B * MB:B * MB + self.work_cap * 8].reshape(self.work_cap, 8)
        tok_splits = h32[B * MB + self.work_cap * 8:]
        from .model_runner import pack_tokens
        q_lens, kv_lens, offs = pack_tokens(out.scheduled, bs, ids, pos, slots, bt)
        rows = [[t] if n == 1 else list(range(t, t + n)) for t, n in zip(offs, q_lens)]
        t = offs[-1] + q_lens[-1] if offs else 0
        N = t
        if N < B:
            ids[N:] = 0
            pos[N:] = 0
            slots[N:] = -1
            bt[len(q_lens), :] = 0
            q_lens.append(B - N)
            kv_lens.append(B - N)
        w, ts, _ = ops.plan_attention_work(q_lens, kv_lens, r.G, True, Hkv=r.model.hkv,
                                           max_splits_cap=self.splits)
        assert w.shape[0] <= self.work_cap
        work[:w.shape[0]] = w
        work[w.shape[0]:] = 0
        tok_splits[:B] = ts[:B]
        return rows

    def upload(self) -> None:
        self.d64.copy_(self.h64, non_blocking=True)
        self.d32.copy_(self.h32, non_blocking=True)
        if self._uploaded is not None:
            self._uploaded.record()
            self._upload_pending = True

    # ------------------------------------------------------------------ capture
    def _body(self):
        r = self.runner
        hidden = r.model.forward(self.batch, r.kv)
        logits = r.model.compute_logits(hidden, fp32=r.config.fp32_lm_head)
        comm = r.comm
        offset = 0
        sharded = comm is not None and comm.ways > 1
        if sharded:
            offset = r.model.vocab_shard(comm.ways, r.shard.head_block)[0]
        ids, vals = ops.argmax_sample(logits, None, None, index_offset=offset)
        if sharded:
            ids = comm.argmax_exchange(ids, vals)
        return ids, hidden

    def capture(self) -> None:
        # warm-up run outside capture (lazy initialisation, autotuned scratch, tensor maps)
        self.upload()
        torch.cuda.synchronize()
        self._body()
        torch.cuda.synchronize()
        n0 = ops.count_launches()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=self.runner.graph_pool()):
            self.ids_out, self.hidden_out = self._body()
        self.launches = ops.count_launches() - n0
        torch.cuda.synchronize()

    def replay(self, prev_ids=None):
        self.upload()
        if prev_ids is not None:
            B = self.bucket
            ops.patch_ids(self.d64[:B], self.d64[3 * B:4 * B], prev_ids)
        self.graph.replay()
        ops.launch_counter.add(self.launches)
        return self.ids_out, self.hidden_out
