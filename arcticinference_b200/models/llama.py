"""Llama-family decoder (Llama 3.x, and the SwiftKV variant) on the engine's own ops.

Weight layout ("rank-major"): with W = TP*SP head-sharding ways, the fused QKV
weight is stored as W consecutive row blocks, block p holding
``[q heads of p | k heads of p | v heads of p]``, and the fused gate/up weight as
blocks ``[gate_p | up_p]``. Consequences:

* the tensor-parallel shard of rank p is a contiguous row view of the full
  matrix, so the shift-parallel (full-TP) mode needs no second copy of the
  weights -- the reference loads a second, TP*SP-sharded model instance for it
  (arctic_inference/vllm/model_runner.py:1692-1714);
* in sequence-parallel mode the QKV GEMM's output columns are already grouped
  by destination rank, which is the "pack" step of the Ulysses all-to-all
  (arctic_inference/vllm/ulysses.py:418-438).

Head ownership: rank (s, t) -- global rank s*TP + t -- owns head block
p = t*SP + s in both modes (arctic_inference/vllm/ulysses.py:222-251), so the
paged KV cache is identical in both modes.

SwiftKV (arctic_inference/vllm/swiftkv/llama_swiftkv.py:220-309): layers
>= num_key_value_layers get their K/V for every token from one fused projection
of ``norm_swiftkv(hidden + residual)`` taken after layer num_key_value_layers-1;
only the tokens that will be sampled continue through those layers.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig


def _rope_type(rs) -> str:
    return (rs or {}).get("rope_type", (rs or {}).get("type", "default")) or "default"


def rope_attention_factor(cfg: ModelConfig) -> float:
    """YaRN scales the rotated queries and keys by an attention factor (cos and sin are
    multiplied by it); here it is folded into the softmax scale as its square. 1 for every
    other rope type."""
    rs = cfg.rope_scaling
    if _rope_type(rs) != "yarn":
        return 1.0
    if rs.get("attention_factor") is not None:
        return float(rs["attention_factor"])
    factor = float(rs["factor"])

    def mscale(scale, m=1.0):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    if rs.get("mscale") and rs.get("mscale_all_dim"):
        return mscale(factor, rs["mscale"]) / mscale(factor, rs["mscale_all_dim"])
    return mscale(factor)


def compute_inv_freq(cfg: ModelConfig, device) -> torch.Tensor:
    """RoPE inverse frequencies [head_dim/2] fp32, with the checkpoint's frequency scaling
    (llama3, linear, yarn) baked in."""
    D = cfg.head_dim
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    rs = cfg.rope_scaling
    kind = _rope_type(rs)
    if kind == "llama3":
        factor = rs["factor"]
        lo, hi = rs["low_freq_factor"], rs["high_freq_factor"]
        old = rs["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor,
                             torch.where(wavelen < old / hi, inv,
                                         (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    elif kind == "linear":
        inv = inv / rs["factor"]
    elif kind == "yarn":
        # high frequencies (many rotations within the original context) keep their value,
        # low ones are interpolated by `factor`, with a linear ramp between the two
        factor = float(rs["factor"])
        old = rs.get("original_max_position_embeddings") or cfg.max_position_embeddings
        fast, slow = rs.get("beta_fast") or 32, rs.get("beta_slow") or 1

        def correction_dim(rotations):
            return D * math.log(old / (rotations * 2 * math.pi)) / (2 * math.log(cfg.rope_theta))

        low, high = correction_dim(fast), correction_dim(slow)
        if rs.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, D - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(D // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        keep = 1 - ramp                                   # 1: extrapolate (unscaled frequency)
        inv = (inv / factor) * (1 - keep) + inv * keep
    elif kind != "default":
        raise NotImplementedError("rope scaling of type %r (supported: llama3, linear, yarn)"
                                  % kind)
    return inv.float().to(device)


@dataclass
class ShardSpec:
    """Where this rank sits in the TP x SP grid and what it stores."""
    tp: int = 1
    sp: int = 1
    tp_rank: int = 0
    sp_rank: int = 0

    @property
    def ways(self) -> int:
        return self.tp * self.sp

    @property
    def head_block(self) -> int:
        """Index p of the head block this rank owns (in both modes)."""
        return self.tp_rank * self.sp + self.sp_rank

    @property
    def stored_blocks(self) -> range:
        """Head blocks whose weights this rank keeps (all blocks of its TP shard)."""
        return range(self.tp_rank * self.sp, (self.tp_rank + 1) * self.sp)


# per-layer tensors in the order every walk over a layer uses (q_norm / k_norm: Qwen3 only;
# bqkv: Qwen2 only, in the row order of wqkv)
LAYER_TENSORS = ("input_norm", "post_norm", "wqkv", "wo", "wgu", "wdown", "q_norm", "k_norm",
                 "bqkv")


class LlamaLayerWeights:
    __slots__ = LAYER_TENSORS + ("wq_swiftkv", "extra")

    def __init__(self):
        self.input_norm = self.post_norm = self.wqkv = self.wo = self.wgu = self.wdown = None
        self.q_norm = self.k_norm = None   # [head_dim] each, shared by all heads of the layer
        self.bqkv = None
        self.wq_swiftkv = None
        self.extra = {}

    def tensors(self):
        """(slot name, tensor) of every tensor this layer holds."""
        for name in LAYER_TENSORS:
            t = getattr(self, name)
            if t is not None:
                yield name, t


class LlamaModel:
    """Weights + forward pass of one rank."""

    def __init__(self, cfg: ModelConfig, shard: Optional[ShardSpec] = None, device="cuda",
                 dtype=torch.bfloat16):
        self.cfg = cfg
        self.shard = shard or ShardSpec()
        self.device = torch.device(device)
        self.dtype = dtype
        W = self.shard.ways
        self.D = cfg.head_dim
        self.Hq, self.Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        if self.Hq % W:
            raise ValueError("query heads must divide by TP*SP")
        self.h = self.Hq // W                      # query heads per block
        self.hkv = max(1, self.Hkv // W)           # kv heads per block
        self.kv_repl = max(1, W // self.Hkv)       # ranks sharing one kv head
        self.blk_rows = (self.h + 2 * self.hkv) * self.D
        self.inter = cfg.intermediate_size
        if self.inter % W:
            raise ValueError("intermediate_size must divide by TP*SP")
        self.inter_blk = self.inter // W
        self.n_stored = len(self.shard.stored_blocks)
        self.layers: list[LlamaLayerWeights] = []
        self.embed = None
        self.norm = None
        self.lm_head = None       # rows of the vocabulary shard this rank scores
        self.norm_swiftkv = None
        self.wkv_swiftkv = None   # fused [L_later * 2*hkv*D (per stored block...), H]
        self.inv_freq = compute_inv_freq(cfg, self.device)
        self.scale = rope_attention_factor(cfg) ** 2 / math.sqrt(self.D)
        self.n_kv_layers = cfg.num_key_value_layers if cfg.is_swiftkv else cfg.num_hidden_layers
        # fp8 weights with per-token activation scales: the norm and SiLU kernels that feed the
        # linear layers emit quantised rows directly (set by quantize_model_fp8)
        self.act_quant = False
        # pipeline parallelism (parallel/pipeline.py): this rank keeps the layers
        # [layer_lo, layer_hi) only; embedding on the first stage, norm + LM head on the last
        self.pp = None
        self.layer_lo, self.layer_hi = 0, cfg.num_hidden_layers

    def set_pipeline(self, pp) -> None:
        if self.cfg.is_swiftkv:
            raise NotImplementedError("pipeline parallelism with SwiftKV models")
        self.pp = pp
        self.layer_lo, self.layer_hi = pp.layer_range(self.cfg.num_hidden_layers)

    # ------------------------------------------------------------------ weights
    def kv_head_of_block(self, p: int) -> range:
        """Global kv heads held by head block p."""
        if self.Hkv >= self.shard.ways:
            return range(p * self.hkv, (p + 1) * self.hkv)
        return range(p // self.kv_repl, p // self.kv_repl + 1)

    def vocab_shard(self, mode_ways: int, index: int) -> tuple[int, int]:
        V = self.cfg.vocab_size
        per = (V + mode_ways - 1) // mode_ways
        per = (per + 7) // 8 * 8
        lo = min(V, index * per)
        return lo, min(V, lo + per)

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        """Random N(0, std) weights in checkpoint (Hugging Face) naming, packed through the
        same path as a real checkpoint: the logical model is the same for every TP x SP
        layout and every rank."""
        from .loader import load_llama_state, random_llama_state
        load_llama_state(self, random_llama_state(self.cfg, seed, std, self.device, self.dtype))

    def num_parameters(self) -> int:
        n = self.embed.numel() + self.norm.numel()
        if self.lm_head is not self.embed:
            n += self.lm_head.numel()
        for lw in self.layers:
            if lw is None:
                continue
            n += sum(t.numel() for _, t in lw.tensors())
        if self.wkv_swiftkv is not None:
            n += self.wkv_swiftkv.numel() + self.norm_swiftkv.numel()
        return n

    def named_tensors(self):
        yield "embed", self.embed
        yield "norm", self.norm
        yield "lm_head", self.lm_head
        if self.norm_swiftkv is not None:
            yield "norm_swiftkv", self.norm_swiftkv
            yield "wkv_swiftkv", self.wkv_swiftkv
        for i, lw in enumerate(self.layers):
            if lw is None:
                continue
            for name, t in lw.tensors():
                yield "layers.%d.%s" % (i, name), t


@dataclass
class ForwardBatch:
    """One step's inputs, identical on every rank (the scheduler runs SPMD)."""
    input_ids: torch.Tensor        # [N] int64
    positions: torch.Tensor        # [N] int64
    slots: torch.Tensor            # [N] int64, -1 for padding
    attn_meta: object              # ops.AttentionMetadata over all N tokens
    logits_indices: torch.Tensor   # [B] int64 rows that are sampled
    num_tokens: int
    mode: str = "tp"               # "sp": Ulysses sequence parallel; "tp": tensor parallel
    # SwiftKV: metadata / positions of the sampled rows only
    sel_attn_meta: object = None
    sel_positions: Optional[torch.Tensor] = None
    # the first ``num_sampled`` selected rows are sampled; further rows are prompt positions
    # whose log-probabilities were asked for: (request, first position, count) per span and
    # the token that follows each such position
    num_sampled: int = 0
    prompt_rows: Optional[list] = None
    prompt_targets: Optional[torch.Tensor] = None


class LlamaForCausalLM(LlamaModel):
    """Adds the forward pass. ``comm`` is a :class:`parallel.Communicator` (None on 1 GPU)."""

    def __init__(self, cfg, shard=None, device="cuda", dtype=torch.bfloat16, comm=None):
        super().__init__(cfg, shard, device, dtype)
        self.comm = comm
        if cfg.qkv_bias and comm is not None and getattr(comm, "fused", False) and comm.sp > 1:
            raise NotImplementedError(
                "a QKV bias (Qwen2) with the fused communicator in sequence-parallel mode: the "
                "scattering GEMM epilogue adds none; use comm_backend='nccl' or tensor "
                "parallelism")

    # --------------------------------------------------------------- shard views
    def _qkv_w(self, lw, mode):
        if mode == "sp" or self.n_stored == 1:
            return lw.wqkv
        i = self.shard.sp_rank
        return lw.wqkv[i * self.blk_rows:(i + 1) * self.blk_rows]

    def _qkv_b(self, lw, mode):
        if lw.bqkv is None or mode == "sp" or self.n_stored == 1:
            return lw.bqkv
        i = self.shard.sp_rank
        return lw.bqkv[i * self.blk_rows:(i + 1) * self.blk_rows]

    def _gu_w(self, lw, mode):
        if mode == "sp" or self.n_stored == 1:
            return lw.wgu
        i = self.shard.sp_rank
        return lw.wgu[i * 2 * self.inter_blk:(i + 1) * 2 * self.inter_blk]

    def _o_w(self, lw, mode):
        if mode == "sp" or self.n_stored == 1:
            return lw.wo
        i = self.shard.sp_rank
        return lw.wo[:, i * self.h * self.D:(i + 1) * self.h * self.D]

    def _down_w(self, lw, mode):
        if mode == "sp" or self.n_stored == 1:
            return lw.wdown
        i = self.shard.sp_rank
        return lw.wdown[:, i * self.inter_blk:(i + 1) * self.inter_blk]

    # ------------------------------------------------------------------- layers
    def _attention_block(self, lw, x, batch, kv, layer, mode, meta, positions, slots,
                         q_only=False):
        """x: normalised hidden rows this rank works on. Returns o_proj output (before the
        tensor-parallel reduction in tp mode)."""
        comm = self.comm
        h, hkv, D = self.h, self.hkv, self.D
        if mode == "sp" and comm is not None and comm.sp > 1:
            # local tokens x all stored head blocks -> all tokens x own head block
            qkv = comm.qkv_scatter_heads(x, lw.wqkv, self.blk_rows, bias=lw.bqkv)
        else:
            w, b = self._qkv_w(lw, mode), self._qkv_b(lw, mode)
            if q_only:
                w = w[: h * D]
            qkv = ops.linear(x, w, bias=b)
        # rows that other ranks scattered into qkv: the first kernel that reads them waits
        wait = comm.take_wait("qkv") if (comm is not None and comm.fused) else None
        if lw.q_norm is not None:
            # Qwen3: every query and key head is normalised over head_dim before RoPE; as the
            # first reader of rows that other ranks stored, this kernel takes the wait
            ops.qk_norm(qkv, lw.q_norm, lw.k_norm, h, 0 if q_only else hkv, D,
                        self.cfg.rms_norm_eps, sync=wait)
            wait = None
        if q_only:
            ops.rope_cache(qkv, positions, None, self.inv_freq, kv.k[layer], kv.v[layer], h, 0, D,
                           sync=wait)
            q = qkv
        else:
            ops.rope_cache(qkv, positions, slots, self.inv_freq, kv.k[layer], kv.v[layer], h, hkv, D,
                           sync=wait)
            q = qkv[:, : h * D]
        if mode == "sp" and comm is not None and comm.sp > 1:
            attn = comm.attention_gather_tokens(q, kv.k[layer], kv.v[layer], meta, h, hkv, D,
                                                self.scale)
        else:
            attn = ops.attention(q, kv.k[layer], kv.v[layer], meta, h, hkv, D, self.scale)
        wait = comm.take_wait("attn") if (comm is not None and comm.fused) else None
        return self._linear_reduce(attn, self._o_w(lw, mode), mode, wait)

    def _mlp_block(self, lw, x, mode):
        gu = ops.linear(x, self._gu_w(lw, mode))
        nblk = self.n_stored if (mode == "sp" or self.n_stored == 1) else 1
        act = ops.silu_mul_blocked(gu, nblk, quant=self.act_quant)
        return self._linear_reduce(act, self._down_w(lw, mode), mode)

    def _linear_reduce(self, x, w, mode, wait=None):
        """Row-parallel linear followed by the reduction its mode needs. With the fused
        communicator the GEMM writes its partial product straight into the symmetric heap; a
        small reduction is then left to the kernel that consumes it (the result is a
        ``PendingReduce`` that ``_norm`` / ``_settle`` take). ``wait``: operand wait for ``x``
        when other ranks store its rows."""
        comm = self.comm
        need = comm is not None and ((mode == "tp" and comm.ways > 1) or
                                     (mode == "sp" and comm.tp > 1))
        if need and comm.fused:
            if comm.folds_reduce(x.shape[0], w.shape[0]):
                return comm.linear_partial(x, w, wait)
            t = ops.linear(x, w, out=comm.reduce_buffer(x.shape[0], w.shape[0]), sync=wait)
        else:
            t = ops.linear(x, w, sync=wait) if wait is not None else ops.linear(x, w)
        return self._reduce(t, mode) if need else t

    def _norm(self, h, weight, residual=None, quant=False):
        """RMSNorm(h (+ residual)) where ``h`` may still be an unreduced row-parallel product."""
        eps = self.cfg.rms_norm_eps
        if isinstance(h, torch.Tensor):
            return ops.rmsnorm(h, weight, eps, residual=residual, quant=quant)
        return self.comm.reduce_rmsnorm(h, weight, eps, residual, quant)

    def _settle(self, h):
        """A plain tensor for ``h`` (reduces it now if it is still pending)."""
        return h if isinstance(h, torch.Tensor) else self.comm.realize(h)

    def _reduce(self, t, mode):
        comm = self.comm
        if comm is None:
            return t
        if mode == "tp":
            return comm.all_reduce_full(t) if comm.ways > 1 else t
        return comm.all_reduce_tp(t) if comm.tp > 1 else t

    def _run_layers(self, lo, hi, h, residual, batch, kv, mode, meta, positions, slots,
                    q_only=False, merged_first=False):
        eps = self.cfg.rms_norm_eps
        aq = self.act_quant
        for l in range(lo, hi):
            lw = self.layers[l]
            if residual is None:
                residual = h
                x = ops.rmsnorm(h, lw.input_norm, eps, quant=aq)
            elif merged_first and l == lo:
                x = ops.rmsnorm(residual, lw.input_norm, eps, quant=aq)
            else:
                x = self._norm(h, lw.input_norm, residual, aq)
            h = self._attention_block(lw, x, batch, kv, l, mode, meta, positions, slots, q_only)
            x = self._norm(h, lw.post_norm, residual, aq)
            h = self._mlp_block(lw, x, mode)
        return h, residual

    # ------------------------------------------------------------------ forward
    def forward(self, batch: ForwardBatch, kv) -> torch.Tensor:
        """Returns the final-norm hidden states of the sampled rows, [B, H]."""
        cfg, comm, mode = self.cfg, self.comm, batch.mode
        eps = cfg.rms_norm_eps
        ids, positions, slots = batch.input_ids, batch.positions, batch.slots
        if comm is not None and comm.fused:
            comm.begin_forward()
        if mode == "sp" and comm is not None and comm.sp > 1:
            ids = comm.local_token_slice(ids)  # contiguous N/SP slice of this rank
        pp = self.pp
        if pp is not None:
            # one stage of the pipeline: take the stream from the stage before, run the local
            # layers, hand it on; only the last stage has logits to offer
            if pp.is_first:
                h, residual = ops.embedding(ids, self.embed), None
            else:
                h, residual = pp.recv_hidden(ids.numel(), cfg.hidden_size, self.dtype, self.device)
            h, residual = self._run_layers(self.layer_lo, self.layer_hi, h, residual, batch, kv,
                                           mode, batch.attn_meta, positions, slots)
            if not pp.is_last:
                pp.send_hidden(h, residual)
                return None
            h = ops.gather_rows(h, batch.logits_indices)
            residual = ops.gather_rows(residual, batch.logits_indices)
            return ops.rmsnorm(h, self.norm, eps, residual=residual)
        h = ops.embedding(ids, self.embed)
        h, residual = self._run_layers(0, self.n_kv_layers, h, None, batch, kv, mode,
                                       batch.attn_meta, positions, slots)
        if not cfg.is_swiftkv:
            h = self._settle(h)
            if mode == "sp" and comm is not None and comm.sp > 1:
                # hand the sampled rows (hidden and residual) to every rank
                h, residual = comm.gather_rows_all(h, residual, batch.logits_indices)
            else:
                h = ops.gather_rows(h, batch.logits_indices)
                residual = ops.gather_rows(residual, batch.logits_indices)
            return ops.rmsnorm(h, self.norm, eps, residual=residual)

        # ---- SwiftKV: one projection produces K/V of all later layers for every token
        if mode == "sp" and comm is not None and comm.sp > 1:
            # later layers run tensor-parallel: every rank needs the normalised state of all
            # tokens (for their K/V) and the residual of the sampled rows
            s, x_sel = comm.swiftkv_boundary(self._settle(h), residual, self.norm_swiftkv, eps,
                                             batch.logits_indices)
        else:
            s = self._norm(h, self.norm_swiftkv, residual)  # residual <- h + residual
            x_sel = ops.gather_rows(residual, batch.logits_indices)
        n_later = cfg.num_hidden_layers - self.n_kv_layers
        wkv = self.wkv_swiftkv
        rows_blk = n_later * 2 * self.hkv * self.D
        if self.n_stored > 1:
            i = self.shard.sp_rank
            wkv = wkv[i * rows_blk:(i + 1) * rows_blk]
        kv_all = ops.linear(s, wkv)
        # one launch rotates K and fills the caches of all later layers
        first = self.n_kv_layers
        tables = kv.pointer_tables(first, n_later) if hasattr(kv, "pointer_tables") else None
        ops.kv_bulk_write(kv_all, positions, slots, self.inv_freq, kv.k[first:first + n_later],
                          kv.v[first:first + n_later], self.hkv, self.D, tables=tables)
        h, residual = self._run_layers(self.n_kv_layers, cfg.num_hidden_layers, None, x_sel, batch,
                                       kv, "tp", batch.sel_attn_meta, batch.sel_positions, None,
                                       q_only=True, merged_first=True)
        return self._norm(h, self.norm, residual)

    def compute_logits(self, hidden: torch.Tensor, fp32: bool = False) -> torch.Tensor:
        """Logits of this rank's vocabulary shard (the full vocabulary on one GPU)."""
        comm = self.comm
        if comm is None or comm.ways == 1:
            w = self.lm_head
        else:
            lo, hi = self.vocab_shard(comm.ways, self.shard.head_block)
            w = self.lm_head[lo:hi]
        if fp32:
            return hidden.float() @ w.float().t()
        return ops.linear(hidden, w)
