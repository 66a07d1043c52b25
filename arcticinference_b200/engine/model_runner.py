"""Turns a :class:`SchedulerOutput` into device work: input staging, the model's
forward pass (eager, or a replayed CUDA graph for decode-shaped steps), logits,
sampling and draft verification.

One runner lives in every rank's process. All ranks build identical inputs
from identical scheduler state, so there is no per-step broadcast of scheduler
output between processes (the reference inherits vLLM's shared-memory message
queue for that: arctic_inference/vllm/ulysses.py:672-796 and worker RPCs).

Shift parallelism (arctic_inference/vllm/model_runner.py:636-662): a step runs
in tensor-parallel mode when it carries at most ``shift_parallel_threshold``
tokens, otherwise in Ulysses sequence-parallel mode; both modes address the
same paged KV cache.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..config import EngineConfig
from ..models.llama import ForwardBatch, LlamaForCausalLM, ShardSpec
from ..utils.tracing import trace_range
from .kv_cache import KVCacheTensors
from .sampler import row_seed
from .scheduler import SchedulerOutput


def pack_tokens(sched, bs: int, ids, pos, slots, bt):
    """Write token ids, positions, cache slots and block-table rows of the scheduled requests
    into the staging arrays. Single-token requests (the bulk of a serving step) are gathered
    in Python lists and written with three vector assignments; only multi-token chunks touch
    numpy per request. Returns (q_lens, kv_lens, token offset of each request)."""
    one_t, one_tok, one_pos, one_slot = [], [], [], []
    q_lens, kv_lens, offs = [], [], []
    t = 0
    for i, s in enumerate(sched):
        r = s.request
        n = s.num_tokens
        st = s.start
        offs.append(t)
        if n == 1:
            one_t.append(t)
            one_tok.append(r.token_at(st))
            one_pos.append(st)
            one_slot.append(r.block_ids[st // bs] * bs + st % bs)
        else:
            known = r.num_tokens
            seq = r.tokens_slice(st, min(st + n, known))
            if len(seq) < n:
                seq = seq + list(r.spec_token_ids[:n - len(seq)])
            ids[t:t + n] = seq
            p = np.arange(st, st + n, dtype=np.int64)
            pos[t:t + n] = p
            blocks = r.block_array().astype(np.int64)
            slots[t:t + n] = blocks[p // bs] * bs + p % bs
        row = r.block_array()
        bt[i, :row.size] = row
        q_lens.append(n)
        kv_lens.append(st + n)
        t += n
    if one_t:
        ids[one_t] = one_tok
        pos[one_t] = one_pos
        slots[one_t] = one_slot
    return q_lens, kv_lens, offs


PLACEHOLDER_TOKEN = -1      # stands for a sampled token the host has not read yet


class PendingStep:
    """A step that has been queued on the device."""

    __slots__ = ("out", "rows", "ids_dev", "hidden", "num_tokens", "mode", "ids_host", "event",
                 "row_of", "logprobs", "prompt_logprobs", "verified")

    def __init__(self, out, rows, ids_dev, hidden, num_tokens, mode):
        self.out, self.rows, self.ids_dev, self.hidden = out, rows, ids_dev, hidden
        self.num_tokens, self.mode = num_tokens, mode
        self.ids_host = None
        self.event = None
        self.row_of = {}
        self.logprobs = None      # (chosen [rows], top values [rows, k], top ids [rows, k])
        self.prompt_logprobs = None   # (values [n], [(request, first position, count)])
        # device-side verification: (accepted tokens [R, max_draft + 1] on the host, -1 padded,
        # the speculator's drafts [R, n] on the host) for the R sampling requests of the step
        self.verified = None


@dataclass
class StepResult:
    new_tokens: dict          # request_id -> list[int]
    drafts: dict              # request_id -> list[int] proposals for the next step
    num_tokens: int
    mode: str
    # request_id -> (log-probabilities of its new tokens, their top alternatives), for the
    # requests that asked for log-probabilities
    logprobs: Optional[dict] = None


def _pinned(n, dtype, device):
    t = torch.empty(n, dtype=dtype)
    if torch.device(device).type == "cuda":
        t = t.pin_memory()
    return t


class ModelRunner:
    def __init__(self, config: EngineConfig, device="cuda", comm=None, shard: ShardSpec = None):
        self.config = config
        self.device = torch.device(device)
        self.comm = comm
        self.shard = shard or ShardSpec()
        mcfg = config.model
        self.model = LlamaForCausalLM(mcfg, self.shard, self.device, torch.bfloat16, comm=comm)
        # a pipeline stage (parallel/pipeline.py): the communicator is then the stage's handle
        self.pp = comm if getattr(comm, "stages", 1) > 1 else None
        if self.pp is not None:
            self.model.set_pipeline(self.pp)
        self.kv: Optional[KVCacheTensors] = None
        self.num_blocks = 0
        self.block_size = config.cache.block_size
        self.sp = config.parallel.sp
        self.shift = config.parallel.enable_shift_parallel
        self.shift_threshold = config.parallel.shift_parallel_threshold
        self.G = self.model.h // self.model.hkv
        self.proposer = None          # set by the engine when speculation is configured
        self.suffix_cache = None
        self._graphs = {}
        self._graph_pool = None
        self._graph_sizes = None
        self._ids_host = [None, None]      # pinned landing buffers for sampled ids
        self._ids_flip = 0
        self.graph_replays = 0
        self.cascade_steps = 0
        self._stage_cap = 0
        self._h_stage = None
        self._stage_events = [None, None]
        self._stage_idx = 0
        self.h2d_bytes = 0
        self.h2d_total = 0
        self.d2h_total = 0
        self.last_step_device_ms = None
        self.mode_counts = {"sp": 0, "tp": 0}
        self.step_timer_events = None
        self.sync_seconds = 0.0       # host time spent blocked on the device for sampled tokens
        self._step_logprobs = None

    # ------------------------------------------------------------------ set-up
    def load_model(self) -> None:
        cfg = self.config
        if cfg.load_format == "dummy" or not cfg.model.name_or_path or \
                cfg.model.name_or_path in __import__("arcticinference_b200.config",
                                                     fromlist=["PRESETS"]).PRESETS:
            self.model.init_random(cfg.seed)
        else:
            from ..models.loader import load_llama_weights
            load_llama_weights(self.model, cfg.model.name_or_path)
        if cfg.model.quantization == "fp8":
            from ..models.quant import quantize_model_fp8
            quantize_model_fp8(self.model, scheme=cfg.model.fp8_scheme)
            if cfg.model.fp8_scheme == "block" and self.comm is not None and \
                    getattr(self.comm, "fused", False):
                self.comm.use_barriers = True   # block-scaled linears carry no signal hooks

    def determine_num_blocks(self) -> int:
        cfg = self.config
        m = self.model
        per_block = KVCacheTensors.bytes_per_block(m.layer_hi - m.layer_lo, m.hkv,
                                                   self.block_size, m.D)
        if cfg.cache.num_gpu_blocks is not None:
            return cfg.cache.num_gpu_blocks
        if self.device.type != "cuda":
            return 512
        free, total = torch.cuda.mem_get_info(self.device)
        # leave room for activations of the largest step and for split-K / split-KV scratch
        reserve = 6 << 30
        budget = int(total * cfg.cache.gpu_memory_utilization) - (total - free) - reserve
        need_max = (cfg.scheduler.max_model_len + self.block_size - 1) // self.block_size
        n = max(budget // per_block, 0)
        if n < need_max + 1:
            raise RuntimeError("not enough GPU memory for one max_model_len sequence "
                               "(%d blocks available, %d needed)" % (n, need_max + 1))
        # cap: block ids are int32 and the tensor maps index blocks with 32-bit coordinates
        return int(min(n, 1 << 22))

    def init_kv_cache(self, num_blocks: int) -> None:
        m = self.model
        self.num_blocks = num_blocks
        self.kv = KVCacheTensors(self.config.model.num_hidden_layers, num_blocks, m.hkv,
                                 self.block_size, m.D, torch.bfloat16, self.device,
                                 layers=range(m.layer_lo, m.layer_hi) if self.pp else None)

    # ------------------------------------------------------------- mode choice
    def choose_mode(self, total_tokens: int) -> str:
        if self.sp <= 1:
            return "tp"
        if self.shift and total_tokens <= self.shift_threshold:
            return "tp"
        return "sp"

    # ---------------------------------------------------------- input staging
    def _stage(self, n_int64: int) -> torch.Tensor:
        """Pinned staging memory for one step's integer inputs. Two buffers alternate and
        each is guarded by an event, so the host never rewrites a buffer whose
        host-to-device copy is still queued (steps that sample nothing do not synchronise)."""
        if n_int64 > self._stage_cap:
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            self._stage_cap = max(n_int64, 2 * self._stage_cap, 1 << 16)
            self._h_stage = [_pinned(self._stage_cap, torch.int64, self.device) for _ in range(2)]
            self._stage_events = [None, None]
            self._stage_idx = 0
        self._stage_idx ^= 1
        ev = self._stage_events[self._stage_idx]
        if ev is not None:
            ev.synchronize()
        return self._h_stage[self._stage_idx][:n_int64]

    def _stage_done(self) -> None:
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._stage_events[self._stage_idx] = ev

    def prepare(self, out: SchedulerOutput):
        """Build the flat batch. Returns (ForwardBatch, rows) where ``rows[i]`` is the list of
        sampled row indices (into logits) of scheduled request i."""
        bs = self.block_size
        sched = out.scheduled
        mode = self.choose_mode(out.total_tokens)
        N = out.total_tokens
        plan = None
        fc = self.config.forest_cascade
        if fc.enabled and mode == "tp" and self.device.type == "cuda":
            from . import forest_cascade as fca
            if fca.gate(fc, [s.num_tokens for s in sched], all(s.samples for s in sched)):
                plan = fca.plan_groups([s.request.block_ids for s in sched],
                                       [s.start for s in sched], bs, fc)
                if plan is not None:
                    sched = [sched[i] for i in plan.order]
                    out.scheduled = sched
                    self.cascade_steps += 1
        pad_to = self.sp if mode == "sp" else 1
        Np = (N + pad_to - 1) // pad_to * pad_to
        n_smp = sum((s.num_draft + 1) if s.samples else 0 for s in sched)
        # prompt log-probabilities: every prompt position of the chunk whose successor is a
        # prompt token is scored too; those rows follow the sampled rows
        prompt_spans = []       # (request, first position, count)
        for s in sched:
            r = s.request
            if r.sampling_params.prompt_logprobs is not None:
                hi = min(s.start + s.num_tokens, r.num_prompt_tokens - 1)
                if hi > s.start:
                    prompt_spans.append((s, s.start, hi - s.start))
        n_sel = n_smp + sum(c for _, _, c in prompt_spans)
        max_blocks = max(len(s.request.block_ids) for s in sched)
        stage = self._stage(3 * Np + n_sel + n_sel)
        h = stage.numpy()
        ids, pos, slots = h[:Np], h[Np:2 * Np], h[2 * Np:3 * Np]
        sel = h[3 * Np:3 * Np + n_sel]
        sel_pos = h[3 * Np + n_sel:3 * Np + 2 * n_sel]
        bt = np.zeros((len(sched), max_blocks), dtype=np.int32)
        q_lens, kv_lens, offs = pack_tokens(sched, bs, ids, pos, slots, bt)
        k = 0
        rows = []
        sel_q_lens = []
        for s, t in zip(sched, offs):
            if s.samples:
                m = s.num_draft + 1
                last = t + s.num_tokens
                if m == 1:
                    sel[k] = last - 1
                    sel_pos[k] = s.start + s.num_tokens - 1
                    rows.append([k])
                else:
                    sel[k:k + m] = np.arange(last - m, last, dtype=np.int64)
                    sel_pos[k:k + m] = np.arange(s.start + s.num_tokens - m, s.start + s.num_tokens,
                                                 dtype=np.int64)
                    rows.append(list(range(k, k + m)))
                sel_q_lens.append(m)
                k += m
            else:
                rows.append([])
                sel_q_lens.append(0)
        prompt_rows = None
        if prompt_spans:
            off_of = {id(s): t for s, t in zip(sched, offs)}
            prompt_rows, targets = [], []
            for s, p0, cnt in prompt_spans:
                t0 = off_of[id(s)] + (p0 - s.start)
                sel[k:k + cnt] = np.arange(t0, t0 + cnt, dtype=np.int64)
                sel_pos[k:k + cnt] = np.arange(p0, p0 + cnt, dtype=np.int64)
                prompt_rows.append((s.request, p0, cnt))
                targets.extend(s.request.prompt_token_ids[p0 + 1:p0 + cnt + 1])
                k += cnt
        if Np > N:
            ids[N:] = 0
            pos[N:] = 0
            slots[N:] = -1
        dev = self.device
        d = stage.to(dev, non_blocking=True)
        self._stage_done()
        self.h2d_bytes = stage.numel() * 8 + bt.nbytes
        self.h2d_total += self.h2d_bytes
        m = self.model
        if Np > N:
            # padding tokens form a sequence of their own that attends to nothing real
            q_lens_a, kv_lens_a = q_lens + [Np - N], kv_lens + [Np - N]
            bt_pad = np.zeros((len(sched) + 1, max_blocks), dtype=np.int32)
            bt_pad[:-1] = bt
            bt_t = ops.upload(bt_pad, dev)
        else:
            q_lens_a, kv_lens_a = q_lens, kv_lens
            bt_t = ops.upload(bt, dev)
        if plan is not None and Np == N:
            from . import forest_cascade as fca
            work, tok_splits, table, max_splits = fca.build_cascade_work(
                plan, q_lens, kv_lens, [s.request.block_ids for s in sched], bs, self.G)
            meta = ops.AttentionMetadata(list(q_lens), list(kv_lens), N)
            meta.work = ops.upload(work, dev)
            meta.tok_splits = ops.upload(tok_splits, dev)
            meta.block_tables = ops.upload(table, dev)
            meta.max_splits, meta.num_work = max_splits, work.shape[0]
            meta.tile_keys = ops.pick_tile_keys(q_lens, self.G)
            meta.o_part = torch.empty(max_splits, N, m.h, m.D, dtype=torch.float32, device=dev)
            meta.lse_part = torch.empty(max_splits, N, m.h, dtype=torch.float32, device=dev)
        else:
            meta = ops.build_attention_metadata(q_lens_a, kv_lens_a, bt_t, self.G, m.h, m.D, dev,
                                                Hkv=m.hkv)
        # the attention work list and split table are uploaded too
        extra = sum(t.numel() * t.element_size() for t in (meta.work, meta.tok_splits)
                    if t is not None)
        self.h2d_bytes += extra
        self.h2d_total += extra
        batch = ForwardBatch(input_ids=d[:Np], positions=d[Np:2 * Np], slots=d[2 * Np:3 * Np],
                             attn_meta=meta, logits_indices=d[3 * Np:3 * Np + n_sel],
                             num_tokens=Np, mode=mode)
        batch.num_sampled = n_smp
        if prompt_rows:
            batch.prompt_rows = prompt_rows
            batch.prompt_targets = ops.upload(np.asarray(targets, dtype=np.int64), dev)
        if self.config.model.is_swiftkv:
            batch.sel_positions = d[3 * Np + n_sel:3 * Np + 2 * n_sel]
            if n_sel:
                sq = [x for x in sel_q_lens if x > 0]
                skv = [kv for kv, x in zip(kv_lens, sel_q_lens) if x > 0]
                keep = [i for i, x in enumerate(sel_q_lens) if x > 0]
                bt_sel = bt_t[ops.upload(np.asarray(keep, dtype=np.int64), dev)].contiguous() \
                    if len(keep) != bt_t.shape[0] else bt_t
                batch.sel_attn_meta = ops.build_attention_metadata(sq, skv, bt_sel, self.G, m.h,
                                                                   m.D, dev, Hkv=m.hkv)
        return batch, rows

    # ---------------------------------------------------------------- sampling
    def _sample(self, logits: torch.Tensor, sched, rows, gathered: bool = False) -> torch.Tensor:
        """Returns int64 [num_rows] token ids on the device. ``gathered``: ``logits`` already
        span the whole vocabulary on every rank."""
        greedy = all(s.request.sampling_params.greedy for s in sched if s.samples)
        plain = all(not s.request.sampling_params.needs_full_logits for s in sched if s.samples)
        comm = self.comm
        sharded = comm is not None and comm.ways > 1 and not gathered
        if plain:
            temps = seeds = None
            if not greedy:
                n = logits.shape[0]
                tv = np.zeros(n, dtype=np.float32)
                sv = np.zeros(n, dtype=np.int64)
                for s, rr in zip(sched, rows):
                    sp = s.request.sampling_params
                    for j, row in enumerate(rr):
                        tv[row] = 0.0 if sp.greedy else sp.temperature
                        sv[row] = row_seed(s.request, j)
                temps = ops.upload(tv, self.device)
                seeds = ops.upload(sv, self.device)
            offset = 0
            if sharded:
                offset = self.model.vocab_shard(comm.ways, self.shard.head_block)[0]
            ids, vals = ops.argmax_sample(logits, temps, seeds, index_offset=offset)
            if sharded:
                ids = comm.argmax_exchange(ids, vals)
            return ids
        # full-distribution path (top-p / top-k / logprobs): framework-level torch ops
        if sharded:
            logits = comm.gather_vocab(logits, self.config.model.vocab_size)
        from .sampler import compute_logprobs, sample_full
        ids = sample_full(logits, sched, rows)
        k = max((s.request.sampling_params.logprobs or 0 for s in sched
                 if s.samples and s.request.sampling_params.logprobs is not None), default=None)
        if k is not None:
            # of the distribution the model put out (before temperature, truncation, grammar)
            self._step_logprobs = compute_logprobs(logits, ids, k)
        return ids

    # ------------------------------------------------------------- CUDA graphs
    def graph_pool(self):
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        return self._graph_pool

    def _decode_graph(self, out: SchedulerOutput):
        """The captured graph for this step, or None when the step must run eagerly."""
        if self.config.enforce_eager or self.device.type != "cuda" or self.pp is not None:
            return None      # (a pipeline stage's step contains point-to-point transfers)
        fc = self.config.forest_cascade
        if fc.enabled and len(out.scheduled) >= fc.min_batch_size:
            return None  # cascade steps plan their own attention work list
        for s in out.scheduled:
            if not s.samples or s.num_tokens != s.num_draft + 1:
                return None
            sp = s.request.sampling_params
            if not sp.greedy or sp.needs_full_logits:
                return None
        from .cuda_graph import DecodeGraph, bucket_for, canonical_sizes
        mode = self.choose_mode(out.total_tokens)
        mult = self.sp if mode == "sp" else 1
        if self._graph_sizes is None:
            self._graph_sizes = canonical_sizes(512)
        bucket = bucket_for((out.total_tokens + mult - 1) // mult, self._graph_sizes)
        if bucket is None:
            return None
        bucket *= mult
        # every sequence needs a block-table row, plus one for the padding sequence
        if len(out.scheduled) + 1 > bucket and out.total_tokens < bucket:
            return None
        key = (mode, bucket)
        g = self._graphs.get(key)
        if g is None:
            g = DecodeGraph(self, mode, bucket)
            g.fill(out)
            try:
                g.capture()
            except Exception as e:  # keep serving eagerly if this shape cannot be captured
                import logging
                logging.getLogger(__name__).warning("CUDA graph capture failed for %s: %s", key, e)
                g = False
            self._graphs[key] = g
        return g or None

    # ------------------------------------------------------------------- step
    def execute(self, out: SchedulerOutput) -> StepResult:
        return self.finish(self.launch(out))

    @staticmethod
    def _logprob_entries(lp_rows, rows, req):
        """(log-probabilities, top alternatives) of the tokens sampled at ``rows``."""
        chosen, topv, topi = lp_rows
        k = req.sampling_params.logprobs or 0
        return ([chosen[j] for j in rows],
                [dict(zip(topi[j][:k], topv[j][:k])) for j in rows])

    @staticmethod
    def _source_rows(out: SchedulerOutput, prev: Optional["PendingStep"]):
        """For every token of this step, the row of ``prev``'s sampled ids that holds it, or
        -1: a request whose newest token is still a placeholder on the host takes it from the
        previous step's device result. None when no token needs that."""
        if prev is None or prev.ids_dev is None:
            return None
        src = np.full(out.total_tokens, -1, dtype=np.int64)
        any_src, t = False, 0
        for s in out.scheduled:
            if s.num_tokens == 1 and s.request.token_at(s.start) == PLACEHOLDER_TOKEN:
                j = prev.row_of.get(id(s.request), -1)
                if j >= 0:
                    src[t] = j
                    any_src = True
            t += s.num_tokens
        return src if any_src else None

    @torch.inference_mode()
    def launch(self, out: SchedulerOutput, prev: Optional["PendingStep"] = None) -> "PendingStep":
        """Queue one step on the device without waiting for its tokens. ``prev`` is the step
        queued before this one whose tokens the host has not read yet: rows of this step that
        feed ``prev``'s sampled token (a placeholder on the host) are patched on the device."""
        g = self._decode_graph(out)
        if g is not None:
            with trace_range("prepare"):
                g.wait_uploaded()
                src_rows = self._source_rows(out, prev)
                rows = g.fill(out, src_rows)
            self.mode_counts[g.mode] += 1
            self.graph_replays += 1
            with trace_range("graph_replay"):
                ids_dev, hidden = g.replay(prev.ids_dev if src_rows is not None else None)
            self.h2d_total += g.h64.numel() * 8 + g.h32.numel() * 4
            pend = PendingStep(out, rows, ids_dev, hidden, g.bucket, g.mode)
            input_sel = g.batch.input_ids       # every row of a decode graph is a sampled row
        else:
            with trace_range("prepare"):
                batch, rows = self.prepare(out)
            self.mode_counts[batch.mode] += 1
            # after prepare(): forest cascade may have put the requests in another order
            src_rows = self._source_rows(out, prev)
            if src_rows is not None:
                n = batch.input_ids.numel()
                if n > src_rows.size:          # rows added to pad the step take no token
                    src_rows = np.concatenate([src_rows, np.full(n - src_rows.size, -1, np.int64)])
                ops.patch_ids(batch.input_ids, ops.upload(src_rows, self.device), prev.ids_dev)
            if batch.logits_indices.numel() == 0:
                # pure prefill chunk: KV only
                self.model.forward(batch, self.kv)
                return PendingStep(out, rows, None, None, batch.num_tokens, batch.mode)
            with trace_range("forward", tokens=batch.num_tokens, mode=batch.mode):
                hidden = self.model.forward(batch, self.kv)
            if self.pp is not None and hidden is None:
                # an earlier pipeline stage: the last stage samples and sends the ids to all
                if batch.prompt_rows:
                    raise NotImplementedError("prompt log-probabilities with pipeline parallelism")
                ids_dev = self.pp.broadcast_ids(None, batch.num_sampled, self.device)
                pend = PendingStep(out, rows, ids_dev, None, batch.num_tokens, batch.mode)
                return self._after_launch(pend, out, rows)
            with trace_range("sample"):
                logits = self.model.compute_logits(hidden, fp32=self.config.fp32_lm_head)
                self._step_logprobs = None
                prompt_lp, gathered = None, False
                if batch.prompt_rows:
                    comm = self.comm
                    if comm is not None and comm.ways > 1:
                        logits = comm.gather_vocab(logits, self.config.model.vocab_size)
                        gathered = True
                    n_s = batch.num_sampled
                    lp = logits[n_s:].float().log_softmax(-1)
                    prompt_lp = lp.gather(1, batch.prompt_targets.unsqueeze(1)).squeeze(1)
                    logits = logits[:n_s]
                ids_dev = self._sample(logits, out.scheduled, rows, gathered) \
                    if logits.shape[0] else None
                if self.pp is not None and ids_dev is not None:
                    ids_dev = self.pp.broadcast_ids(ids_dev.contiguous(), ids_dev.numel(), self.device)
            pend = PendingStep(out, rows, ids_dev, hidden, batch.num_tokens, batch.mode)
            pend.logprobs, self._step_logprobs = self._step_logprobs, None
            input_sel = None
            if self.proposer is not None and ids_dev is not None:
                input_sel = batch.input_ids[batch.logits_indices[:batch.num_sampled]]
            if prompt_lp is not None:
                pend.prompt_logprobs = (prompt_lp, batch.prompt_rows)
        return self._after_launch(pend, out, rows, input_sel)

    def _after_launch(self, pend, out, rows, input_sel=None):
        """Start the step's tokens on their way to the host (and, with a speculator, verify
        and draft on the device)."""
        # the device result may be overwritten by the next replay of the same graph: take the
        # host copy now, read it in finish()
        if self.device.type == "cuda" and pend.ids_dev is not None:
            host = self._ids_host[self._ids_flip]
            if host is None or host.numel() < pend.ids_dev.numel():
                host = torch.empty(max(pend.ids_dev.numel(), 4096), dtype=torch.int64, pin_memory=True)
                self._ids_host[self._ids_flip] = host
            pend.ids_host = host[:pend.ids_dev.numel()]
            pend.ids_host.copy_(pend.ids_dev, non_blocking=True)
            if self.proposer is not None:
                self._verify_and_draft(pend, input_sel)
            pend.event = torch.cuda.Event()
            pend.event.record()
            self._ids_flip ^= 1
        elif self.proposer is not None and pend.ids_dev is not None:
            self._verify_and_draft(pend, input_sel)
        pend.row_of = {id(s.request): rr[0] for s, rr in zip(out.scheduled, rows) if rr}
        return pend

    def _verify_and_draft(self, pend: "PendingStep", input_sel: torch.Tensor) -> None:
        """Accept drafts and draft again without leaving the stream: one kernel compares every
        request's draft tokens with the tokens the model produced after them, the speculator
        then runs from the hidden state at each request's last accepted row and the token that
        follows it, and both results travel to pinned host memory behind the step's tokens.
        The host reads them in ``finish`` after the one synchronisation it does anyway (the
        reference verifies in its rejection sampler and feeds the proposer from device tensors:
        arctic_inference/vllm/model_runner.py:1008-1023, spec_dec/arctic_proposer.py:130-209)."""
        from ..ops import spec_ops
        sched, rows = pend.out.scheduled, pend.rows
        live = [(s, rr) for s, rr in zip(sched, rows) if s.samples]
        R = len(live)
        if R == 0:
            return
        meta = np.empty(2 * R, dtype=np.int32)
        meta[:R] = [rr[0] for _, rr in live]
        meta[R:] = [s.num_draft for s, _ in live]
        max_draft = int(meta[R:].max())
        meta_dev = ops.upload(meta, self.device)
        self.h2d_total += meta.nbytes
        _, next_tok, sel_row, out_tokens = spec_ops.verify_greedy(
            input_sel, pend.ids_dev, meta_dev[:R], meta_dev[R:], max_draft)
        cfg = self.config.speculative
        n_predict = cfg.num_speculative_tokens or self.proposer.n_predict
        cuda = pend.hidden.is_cuda
        h = ops.gather_rows(pend.hidden, sel_row) if cuda else pend.hidden[sel_row]
        drafts = self.proposer.propose(h, next_tok, n_predict)
        out_host = torch.empty(out_tokens.shape, dtype=torch.int64, pin_memory=cuda)
        out_host.copy_(out_tokens, non_blocking=True)
        drafts_host = torch.empty(drafts.shape, dtype=torch.int64, pin_memory=cuda)
        drafts_host.copy_(drafts, non_blocking=True)
        self.d2h_total += (out_tokens.numel() + drafts.numel()) * 8
        pend.verified = (out_host, drafts_host)

    @torch.inference_mode()
    def finish(self, pend: "PendingStep") -> StepResult:
        """Read the step's tokens (synchronises with the device) and turn them into per-request
        token lists; propose drafts for the next step when speculation is on."""
        new_tokens: dict = {}
        drafts: dict = {}
        sched, rows = pend.out.scheduled, pend.rows
        if pend.prompt_logprobs is not None:
            vals, spans = pend.prompt_logprobs
            vals = vals.tolist()            # synchronises the step
            o = 0
            for req, p0, cnt in spans:
                if req.prompt_logprobs is None:
                    req.prompt_logprobs = [None] * req.num_prompt_tokens
                # the value at index p + 1 is log P(prompt[p + 1] | prompt[:p + 1])
                req.prompt_logprobs[p0 + 1:p0 + cnt + 1] = vals[o:o + cnt]
                o += cnt
        if pend.ids_dev is None:
            return StepResult(new_tokens, drafts, pend.num_tokens, pend.mode)
        with trace_range("sync_tokens"):
            if pend.ids_host is not None:
                t0 = time.perf_counter()
                pend.event.synchronize()
                self.sync_seconds += time.perf_counter() - t0
                ids = pend.ids_host.tolist()
            else:
                ids = pend.ids_dev.tolist()  # device -> host; synchronises the step
        self.d2h_total += len(ids) * 8
        accepted_rows = []
        lp_rows = None
        logprobs: Optional[dict] = None
        if pend.logprobs is not None:
            chosen, topv, topi = (t.tolist() for t in pend.logprobs)
            lp_rows = (chosen, topv, topi)
            logprobs = {}
        arctic = None
        if pend.verified is not None:
            # the device compared drafts with targets already: its rows are the accepted
            # tokens and the one that follows them
            out_host, drafts_host = pend.verified
            arctic = drafts_host.tolist()
            live = [(s, rr) for s, rr in zip(sched, rows) if s.samples]
            for (s, rr), row in zip(live, out_host.tolist()):
                r = s.request
                toks = row[:s.num_draft + 1]
                if toks[-1] < 0:
                    toks = toks[:toks.index(-1)]
                new_tokens[r.request_id] = toks
                accepted_rows.append(rr[len(toks) - 1])
                if lp_rows is not None and r.sampling_params.logprobs is not None:
                    logprobs[r.request_id] = self._logprob_entries(lp_rows, rr[:len(toks)], r)
        for s, rr in zip(sched, rows):
            if not s.samples or pend.verified is not None:
                continue
            r = s.request
            if len(rr) == 1:
                new_tokens[r.request_id] = [ids[rr[0]]]
                accepted_rows.append(rr[0])
                if lp_rows is not None and r.sampling_params.logprobs is not None:
                    logprobs[r.request_id] = self._logprob_entries(lp_rows, rr[:1], r)
                continue
            target = [ids[j] for j in rr]
            toks = [target[0]]
            if s.num_draft:
                draft = r.spec_token_ids[:s.num_draft]
                for j, dtok in enumerate(draft):
                    if dtok != target[j]:
                        break
                    toks.append(target[j + 1])
            new_tokens[r.request_id] = toks
            accepted_rows.append(rr[len(toks) - 1])
            if lp_rows is not None and r.sampling_params.logprobs is not None:
                logprobs[r.request_id] = self._logprob_entries(lp_rows, rr[:len(toks)], r)
        if self.proposer is not None or self.suffix_cache is not None:
            from ..spec_decode.propose import propose_drafts
            with trace_range("draft"):
                drafts = propose_drafts(self, sched, rows, new_tokens, pend.hidden, accepted_rows,
                                        arctic=arctic)
        return StepResult(new_tokens, drafts, pend.num_tokens, pend.mode, logprobs)
