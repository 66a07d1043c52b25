"""Embedding engine: token lists in, pooled fp32 vectors out.

One engine owns one GPU. Requests are split into packed batches under a token budget
(sequences sorted by length so that the attention tiles of a batch are evenly filled). Two
sets of pinned staging buffers alternate: all copies are asynchronous, so the host packs and
enqueues batch i+1 while batch i computes and only collects a batch's embeddings when its
staging set comes round again.
:class:`AsyncEmbeddingEngine` adds a worker thread that merges the sequences of concurrent
callers into common batches (the reference gets the equivalent from vLLM's scheduler behind
``AsyncLLMEngine.encode``: arctic_inference/embedding/replica.py:101-128).
"""

from __future__ import annotations

import asyncio
import queue
import threading
import time
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from ..config import ModelConfig
from ..models.bert import BertEncoder
from ..utils.tokenizer import get_tokenizer


@dataclass
class EmbeddingStats:
    requests: int = 0
    sequences: int = 0
    tokens: int = 0
    batches: int = 0
    busy_seconds: float = 0.0
    h2d_bytes: int = 0
    d2h_bytes: int = 0


class _Staging:
    """Pinned host buffers + device buffers of one in-flight batch."""

    def __init__(self, max_tokens: int, max_seqs: int, hidden: int, device):
        pin = device.type == "cuda"
        self.ids = torch.empty(2, max_tokens, dtype=torch.int64, pin_memory=pin)     # ids | positions
        self.starts = torch.empty(max_seqs + 1, dtype=torch.int64, pin_memory=pin)
        self.out = torch.empty(max_seqs, hidden, dtype=torch.float32, pin_memory=pin)
        self.d_ids = torch.empty(2, max_tokens, dtype=torch.int64, device=device)
        self.d_starts = torch.empty(max_seqs + 1, dtype=torch.int64, device=device)
        self.d_out = torch.empty(max_seqs, hidden, dtype=torch.float32, device=device)
        self.done = torch.cuda.Event() if pin else None
        self.pending = None      # (indices, n_seqs) of the batch whose result sits in `out`


class EmbeddingEngine:
    def __init__(self, model: str = "bert-base", device=None, dtype=torch.bfloat16,
                 max_num_batched_tokens: int = 16384, max_num_seqs: int = 2048,
                 pooling: Optional[str] = None, normalize: Optional[bool] = None, seed: int = 0,
                 model_config: Optional[ModelConfig] = None):
        self.cfg = model_config or ModelConfig.from_pretrained(model)
        if not self.cfg.is_encoder:
            raise ValueError("%s is not an encoder model" % model)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if self.device.type == "cpu":
            dtype = torch.float32 if dtype is None else dtype
        self.model_name = model
        self.pooling = pooling or self.cfg.pooling
        self.normalize = self.cfg.normalize if normalize is None else normalize
        self.max_len = self.cfg.max_position_embeddings
        self.max_tokens = max(max_num_batched_tokens, self.max_len)
        self.max_seqs = max_num_seqs
        self.encoder = BertEncoder(self.cfg, self.device, dtype)
        import os
        if model in ("bert-base", "bert-tiny") or not os.path.isdir(model):
            self.encoder.init_random(seed)
        else:
            self.encoder.load_pretrained(model)
        self.tokenizer = get_tokenizer(model, self.cfg.vocab_size)
        self.stats = EmbeddingStats()
        self._stage = [_Staging(self.max_tokens, self.max_seqs, self.cfg.hidden_size, self.device)
                       for _ in range(2)]
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ batching
    def tokenize(self, prompts: Sequence) -> list:
        out = []
        for p in prompts:
            if isinstance(p, str):
                ids = self.tokenizer.encode(p)
                ids = list(ids["input_ids"]) if isinstance(ids, dict) else list(ids)
            else:
                ids = p
            a = np.asarray(ids, dtype=np.int64).reshape(-1)
            if a.size > self.max_len:
                # cut like a tokenizer with truncation does: the closing [SEP] stays
                sep = getattr(self.tokenizer, "sep_token_id", None)
                keep_last = isinstance(p, str) and sep is not None and a[-1] == sep
                a = np.concatenate([a[: self.max_len - 1], a[-1:]]) if keep_last else a[: self.max_len]
            out.append(a if a.size else np.zeros(1, dtype=np.int64))
        return out

    def plan_batches(self, lens: Sequence[int]) -> list:
        """Indices grouped into batches: longest first, each batch within the token and
        sequence budgets."""
        order = sorted(range(len(lens)), key=lambda i: -lens[i])
        batches, cur, tok = [], [], 0
        for i in order:
            if cur and (tok + lens[i] > self.max_tokens or len(cur) >= self.max_seqs):
                batches.append(cur)
                cur, tok = [], 0
            cur.append(i)
            tok += lens[i]
        if cur:
            batches.append(cur)
        return batches

    # ------------------------------------------------------------------ execution
    def _fill(self, st: _Staging, seqs: list) -> tuple:
        ids, starts = st.ids.numpy(), st.starts.numpy()
        lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=len(seqs))
        S = len(seqs)
        starts[0] = 0
        np.cumsum(lens, out=starts[1:S + 1])
        T = int(starts[S])
        np.concatenate(seqs, out=ids[0, :T])
        # position of token t inside its sequence = t - start of that sequence
        ids[1, :T] = np.arange(T) - np.repeat(starts[:S], lens)
        return T, S

    def _drain(self, st: _Staging, result: np.ndarray) -> None:
        if st.pending is None:
            return
        idx, n = st.pending
        if st.done is not None:
            st.done.synchronize()
        result[idx] = st.out[:n].numpy()
        st.pending = None

    def encode(self, prompts: Sequence, pooling: Optional[str] = None,
               normalize: Optional[bool] = None) -> np.ndarray:
        """Embeddings fp32 [len(prompts), hidden]. ``prompts``: strings or token-id lists."""
        seqs = self.tokenize(prompts)
        H = self.cfg.hidden_size
        result = np.empty((len(seqs), H), dtype=np.float32)
        if not seqs:
            return result
        t0 = time.perf_counter()
        with self._lock:
            batches = self.plan_batches([len(s) for s in seqs])
            cuda = self.device.type == "cuda"
            for b, idx in enumerate(batches):
                st = self._stage[b & 1]
                self._drain(st, result)                 # the batch two steps back
                T, S = self._fill(st, [seqs[i] for i in idx])
                lens = [len(seqs[i]) for i in idx]
                if cuda:
                    st.d_ids[:, :T].copy_(st.ids[:, :T], non_blocking=True)
                    st.d_starts[:S + 1].copy_(st.starts[:S + 1], non_blocking=True)
                    d_ids, d_starts, d_out = st.d_ids, st.d_starts, st.d_out
                else:
                    d_ids, d_starts, d_out = st.ids, st.starts, None
                out = self.encoder.embed(d_ids[0, :T], d_ids[1, :T], lens, d_starts[:S + 1],
                                         pooling=pooling or self.pooling,
                                         normalize=self.normalize if normalize is None else normalize,
                                         out=None if d_out is None else d_out[:S])
                if cuda:
                    st.out[:S].copy_(d_out[:S], non_blocking=True)
                    st.done.record()
                else:
                    st.out[:S].copy_(out)
                st.pending = (idx, S)
                self.stats.batches += 1
                self.stats.tokens += T
                self.stats.h2d_bytes += 16 * T + 8 * (S + 1)
                self.stats.d2h_bytes += 4 * S * H
            for st in self._stage:
                self._drain(st, result)
            if cuda:
                from .. import ops
                ops.check_status()
        self.stats.requests += 1
        self.stats.sequences += len(seqs)
        self.stats.busy_seconds += time.perf_counter() - t0
        return result


@dataclass
class _Work:
    seqs: list
    future: "asyncio.Future"
    loop: "asyncio.AbstractEventLoop"
    request_id: str = ""
    aborted: bool = False


class AsyncEmbeddingEngine:
    """Worker thread in front of an :class:`EmbeddingEngine`: concurrent ``encode`` calls are
    merged into shared batches; a request can be aborted until the worker has picked it up."""

    def __init__(self, engine: EmbeddingEngine, max_wait_ms: float = 1.0):
        self.engine = engine
        self.max_wait = max_wait_ms / 1e3
        self._q: "queue.Queue[Optional[_Work]]" = queue.Queue()
        self._inflight: dict = {}
        self._thread = threading.Thread(target=self._run, name="embedding-worker", daemon=True)
        self._stopped = False
        self._thread.start()

    @property
    def pending(self) -> int:
        return self._q.qsize()

    def _run(self) -> None:
        while True:
            w = self._q.get()
            if w is None:
                return
            group = [w]
            deadline = time.perf_counter() + self.max_wait
            tokens = sum(len(s) for s in w.seqs)
            while tokens < self.engine.max_tokens:
                try:
                    nxt = self._q.get(timeout=max(0.0, deadline - time.perf_counter()))
                except queue.Empty:
                    break
                if nxt is None:
                    self._q.put(None)
                    break
                group.append(nxt)
                tokens += sum(len(s) for s in nxt.seqs)
            live = [g for g in group if not g.aborted]
            for g in group:
                self._inflight.pop(g.request_id, None)
                if g.aborted:
                    g.loop.call_soon_threadsafe(_set_exception, g.future, RuntimeError("aborted"))
            if not live:
                continue
            try:
                flat = [s for g in live for s in g.seqs]
                emb = self.engine.encode(flat)
                o = 0
                for g in live:
                    n = len(g.seqs)
                    g.loop.call_soon_threadsafe(_set_result, g.future, emb[o:o + n])
                    o += n
            except Exception as e:  # noqa: BLE001 - forwarded to the callers
                for g in live:
                    g.loop.call_soon_threadsafe(_set_exception, g.future, e)

    async def encode(self, prompts: Sequence, request_id: str = "") -> np.ndarray:
        if self._stopped:
            raise RuntimeError("engine stopped")
        loop = asyncio.get_running_loop()
        w = _Work(self.engine.tokenize(prompts), loop.create_future(), loop, request_id)
        if request_id:
            self._inflight[request_id] = w
        self._q.put(w)
        return await w.future

    def abort(self, request_id: str) -> bool:
        w = self._inflight.get(request_id)
        if w is None:
            return False
        w.aborted = True
        return True

    def stop(self) -> None:
        if not self._stopped:
            self._stopped = True
            self._q.put(None)
            self._thread.join(timeout=10)


def _set_result(fut, value):
    if not fut.done():
        fut.set_result(value)


def _set_exception(fut, exc):
    if not fut.done():
        fut.set_exception(exc)
