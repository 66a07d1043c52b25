"""Arctic draft models: the MLP speculator and the LSTM ("sum_lstm") speculator.

Both turn the target model's last hidden state at the last accepted token, plus the
newly sampled token, into ``n_predict`` further draft tokens, one head per token
(arctic_inference/vllm/spec_dec/arctic_speculator.py:122-459 and :462-1067).

MLP head i:   state = GELU(LN_i(W_proj,i . prev + (emb_w / state_w) . E_i[tok]))
LSTM head i:  gates = W_projs[min(i,1)] . prev + (emb_w / state_w) . repeat4(E_forget[tok])
              c = c_prev . sig(f) + GELU(LN_cell(g_c)) . sig(i);  state = GELU(LN_state(c)) . sig(o)
then          logits = W_head . state,  tok = argmax,  prev = state
with state_w = 0.5 ** (0.5 / n_predict), emb_w = sqrt((1 - state_w^2) * inner_dim / 2) and, when
``scale_input`` is set, prev_0 = RMSNorm(hidden) / sqrt(2).

Each step is three launches: the projection GEMM, one fused cell kernel (embedding gather +
gate sum + both normalisations + activations, ``csrc/speculator.cu``) and the LM-head GEMM,
followed by the arg-max kernel. On a multi-GPU engine every rank holds the whole draft model
and computes the same draft: the speculator is small next to 180 GB of HBM, and replication
removes the embedding all-reduce and the top-1 all-gather the reference needs per head
(arctic_inference/vllm/spec_dec/vocab_parallel_embedding.py:437,
arctic_speculator.py:332-342).

Checkpoint format: ``config.json`` with ``n_predict, vocab_size, emb_dim, inner_dim, proj_dim,
input_hidden_dim, tie_weights, tie_lstm_embs, scale_input, method``; dims may be dotted strings
("4096.4096"). Weight names may carry a ``speculator.`` prefix. LSTM gate projections may be
stored fused (``projs.N.weight``) or split (``forget_proj/input_proj/output_proj/cell_proj.N``),
fused here in the order f, i, o, c (arctic_speculator.py:1027-1067).
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Iterable, Optional

import torch

from .. import ops
from ..ops import spec_ops


def _first_dim(v) -> int:
    if isinstance(v, str):
        return int(v.split(".")[0])
    if isinstance(v, (list, tuple)):
        return int(v[0])
    return int(v)


@dataclass
class SpeculatorConfig:
    n_predict: int = 3
    vocab_size: int = 128256
    emb_dim: int = 4096
    inner_dim: int = 4096
    proj_dim: int = 4096
    input_hidden_dim: int = 4096
    tie_weights: bool = True
    tie_lstm_embs: bool = True
    scale_input: bool = True
    method: str = "sum_lstm"      # "mlp" | "sum_rnn" | "sum_lstm"
    num_lookahead_tokens: Optional[int] = None
    base_model_archs: Optional[list] = None
    architecture: str = "ArcticLSTMSpeculatorPreTrainedModel"

    @classmethod
    def from_dict(cls, d: dict) -> "SpeculatorConfig":
        archs = d.get("architectures") or ["MLPSpeculatorPreTrainedModel"]
        arch = archs[0]
        method = d.get("method")
        if method is None:
            method = "sum_rnn" if "LSTM" in arch or "MLPVariant" in arch else "mlp"
        emb = _first_dim(d.get("emb_dim", 4096))
        inner = _first_dim(d.get("inner_dim", 0)) or emb
        return cls(n_predict=int(d.get("n_predict", 3)), vocab_size=int(d["vocab_size"]),
                   emb_dim=emb, inner_dim=inner, proj_dim=_first_dim(d.get("proj_dim", inner)) or inner,
                   input_hidden_dim=int(d.get("input_hidden_dim", emb)),
                   tie_weights=bool(d.get("tie_weights", False)),
                   tie_lstm_embs=bool(d.get("tie_lstm_embs", True)),
                   scale_input=bool(d.get("scale_input", False)), method=method,
                   num_lookahead_tokens=d.get("num_lookahead_tokens"),
                   base_model_archs=d.get("base_model_archs"), architecture=arch)

    @classmethod
    def from_pretrained(cls, path: str) -> "SpeculatorConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))


class ArcticSpeculator:
    """Weights + the n-head proposal loop of either speculator type."""

    LN_EPS = 1e-6

    def __init__(self, cfg: SpeculatorConfig, device="cuda", dtype=torch.bfloat16):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_predict = cfg.n_predict
        self.lstm = cfg.method == "sum_lstm"
        self.state_weight = 0.5 ** (0.5 / cfg.n_predict)
        self.emb_weight = math.sqrt((1 - self.state_weight ** 2) * (cfg.inner_dim / 2))
        self.alpha = self.emb_weight / self.state_weight
        self.w: dict[str, torch.Tensor] = {}

    # ----------------------------------------------------------------- weight indexing
    def _idx(self, kind: str, i: int) -> int:
        if not self.cfg.tie_weights:
            return i
        return min(i, 1) if kind == "proj" else 0

    def expected_tensors(self) -> dict:
        c = self.cfg
        shapes = {}
        n = c.n_predict
        if self.lstm:
            shapes["forget_emb.0.weight"] = (c.vocab_size, c.emb_dim)
            if not c.tie_lstm_embs:
                for g in ("input", "output", "cell"):
                    shapes["%s_emb.0.weight" % g] = (c.vocab_size, c.emb_dim)
            shapes["projs.0.weight"] = (4 * c.proj_dim, c.input_hidden_dim)
            if n > 1:
                shapes["projs.1.weight"] = (4 * c.proj_dim, c.inner_dim)
            for ln in ("cell_ln", "state_ln"):
                shapes["%s.0.weight" % ln] = (c.inner_dim,)
                shapes["%s.0.bias" % ln] = (c.inner_dim,)
            shapes["head.0.weight"] = (c.vocab_size, c.inner_dim)
        else:
            heads = range(n)
            for i in heads:
                if self._idx("emb", i) == i:
                    shapes["emb.%d.weight" % i] = (c.vocab_size, c.inner_dim)
                    shapes["ln.%d.weight" % i] = (c.inner_dim,)
                    shapes["ln.%d.bias" % i] = (c.inner_dim,)
                    shapes["head.%d.weight" % i] = (c.vocab_size, c.inner_dim)
                if self._idx("proj", i) == i:
                    shapes["proj.%d.weight" % i] = (c.inner_dim,
                                                    c.input_hidden_dim if i == 0 else c.inner_dim)
        return shapes

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        gen = torch.Generator(device=self.device)
        for k, (name, shape) in enumerate(sorted(self.expected_tensors().items())):
            gen.manual_seed(seed * 7919 + 31 * k + 5)
            if name.endswith("ln.0.weight") or (".weight" in name and len(shape) == 1):
                t = torch.ones(shape, device=self.device, dtype=self.dtype)
            elif name.endswith(".bias"):
                t = torch.zeros(shape, device=self.device, dtype=self.dtype)
            else:
                t = (torch.randn(*shape, generator=gen, device=self.device,
                                 dtype=torch.float32) * std).to(self.dtype)
            self.w[name] = t

    def load_state(self, state: Iterable) -> None:
        """(name, tensor) pairs in checkpoint naming (optionally prefixed ``speculator.``)."""
        split: dict[tuple, dict] = {}
        for name, t in state:
            if name.startswith("speculator."):
                name = name[len("speculator."):]
            parts = name.split(".")
            if parts[0] in ("forget_proj", "input_proj", "output_proj", "cell_proj"):
                split.setdefault((parts[1], parts[2]), {})[parts[0]] = t
                continue
            self.w[name] = t.to(device=self.device, dtype=self.dtype).contiguous()
        for (idx, kind), gates in split.items():
            fused = torch.cat([gates[g] for g in ("forget_proj", "input_proj", "output_proj",
                                                  "cell_proj")], 0)
            self.w["projs.%s.%s" % (idx, kind)] = fused.to(device=self.device,
                                                           dtype=self.dtype).contiguous()
        if self.lstm and not self.cfg.tie_lstm_embs:
            self.w["forget_emb.0.weight"] = torch.cat(
                [self.w.pop("%s_emb.0.weight" % g) if g != "forget" else self.w["forget_emb.0.weight"]
                 for g in ("forget", "input", "output", "cell")], 1).contiguous()
        missing = [k for k in self.expected_tensors() if k not in self.w and "_emb" not in k[1:]]
        if missing:
            raise ValueError("speculator checkpoint lacks %s" % missing[:6])

    def load_pretrained(self, path: str) -> None:
        from .loader import iter_safetensors_dir
        self.load_state(iter_safetensors_dir(path))

    def quantize_fp8(self) -> int:
        """Store the projections and LM heads as fp8 with one scale per output feature
        (activations are quantised per token on the way in; embeddings and norms stay bf16);
        matrices whose inner dimension is not a multiple of 16 are left alone. Returns the
        number of tensors converted. (Reference: arctic_inference/vllm/spec_dec/fp8.py:140-309
        quantises the same linears of its speculators.)"""
        from .quant import quantize_weight_fp8_row
        n = 0
        for k, t in list(self.w.items()):
            if not isinstance(t, torch.Tensor) or t.dim() != 2:
                continue
            if not (k.startswith("proj") or k.startswith("head")):
                continue
            if t.shape[0] % 8 or t.shape[1] % 16:
                continue
            self.w[k] = quantize_weight_fp8_row(t)
            n += 1
        return n

    # ---------------------------------------------------------------- vocabulary shards
    def shard_heads(self, comm) -> bool:
        """Keep only this rank's slice of every LM head's vocabulary rows: each rank then
        streams 1/W of the head per draft token and the ranks exchange one (value, token)
        candidate per row (``comm.argmax_exchange``, 16 bytes per row per rank; the
        reference's top-1 exchange: arctic_speculator.py:328-342). Embeddings stay replicated
        (a row gather, no reduction to pay for). Returns False, leaving the heads whole, when
        the vocabulary does not split into multiples of 16 rows."""
        W = comm.ways
        V = self.cfg.vocab_size
        if W <= 1 or V % (16 * W):
            return False
        per = V // W
        off = comm.rank * per
        for k in [k for k in self.w if k.startswith("head")]:
            t = self.w[k]
            if isinstance(t, torch.Tensor):
                self.w[k] = t[off:off + per].clone()
            else:                                   # a quantised head: slice codes and scales
                self.w[k] = t[off:off + per]
        self.tp_comm, self.tp_offset, self.tp_rows = comm, off, per
        return True

    QHEAD_MAX_BATCH = 32

    def make_qheads(self) -> int:
        """Keep an fp8 copy (one scale per vocabulary row) of every bf16 LM head beside the
        head itself; drafts for at most ``QHEAD_MAX_BATCH`` requests read the fp8 copy, where
        the head is a pure weight stream and half the bytes is half the time, larger batches
        the bf16 head (the reference's rule: arctic_speculator.py:324-325, its ``qhead`` is
        built at :519-535). Returns the number of copies made."""
        from .quant import quantize_weight_fp8_row
        self.qhead = {}
        for k, t in self.w.items():
            if k.startswith("head") and isinstance(t, torch.Tensor) and t.dim() == 2 and \
                    t.is_cuda and t.shape[0] % 8 == 0 and t.shape[1] % 16 == 0:
                self.qhead[k] = quantize_weight_fp8_row(t)
        return len(self.qhead)

    def _head(self, key: str, batch: int):
        q = getattr(self, "qhead", None)
        if q and batch <= self.QHEAD_MAX_BATCH and key in q:
            return q[key]
        return self.w[key]

    def weight_slots(self):
        """(owner, key) pairs of every tensor, for sleep / wake and weight sync."""
        slots = [(self.w, k) for k in list(self.w)]
        q = getattr(self, "qhead", None)
        if q:
            slots += [(q, k) for k in list(q)]
        return slots

    def num_parameters(self) -> int:
        return sum(t.numel() for t in self.w.values())

    # ------------------------------------------------------------------------ forward
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512)

    def propose(self, hidden: torch.Tensor, tokens: torch.Tensor,
                n_predict: Optional[int] = None) -> torch.Tensor:
        """hidden: [B, input_hidden_dim] target hidden states at the last accepted tokens;
        tokens: [B] int64 the tokens just sampled. Returns draft tokens int64 [B, n_predict].

        On a GPU the whole n-head loop (4n + 1 small kernels) runs as one CUDA graph per padded
        batch size, replayed on static input buffers (the reference captures the same loop:
        arctic_inference/vllm/spec_dec/arctic_speculator.py:350-420,923-981);
        ``ARCTIC_B200_SPEC_GRAPH=0`` or a capture in progress runs it eagerly."""
        n = n_predict or self.n_predict
        B = hidden.shape[0]
        if (hidden.is_cuda and self.use_graph and 0 < B <= self.GRAPH_BUCKETS[-1]
                and not torch.cuda.is_current_stream_capturing()):
            return self._propose_graphed(hidden, tokens, n)
        return self._propose(hidden, tokens, n)

    @property
    def use_graph(self) -> bool:
        import os
        return os.environ.get("ARCTIC_B200_SPEC_GRAPH", "1") != "0"

    def _propose_graphed(self, hidden, tokens, n):
        B = hidden.shape[0]
        bucket = next(b for b in self.GRAPH_BUCKETS if b >= B)
        key = (bucket, n, hidden.shape[1])
        graphs = self.__dict__.setdefault("_graphs", {})
        g = graphs.get(key)
        if g is None:
            h_buf = torch.zeros(bucket, hidden.shape[1], dtype=hidden.dtype, device=hidden.device)
            t_buf = torch.zeros(bucket, dtype=torch.int64, device=hidden.device)
            self._propose(h_buf, t_buf, n)          # warm-up outside the capture
            torch.cuda.synchronize(hidden.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._propose(h_buf, t_buf, n)
            g = graphs[key] = (graph, h_buf, t_buf, out)
        graph, h_buf, t_buf, out = g
        h_buf[:B].copy_(hidden)
        t_buf[:B].copy_(tokens)
        graph.replay()
        # the buffers are rewritten by the next call: hand out a copy
        return out[:B].clone()

    def _propose(self, hidden: torch.Tensor, tokens: torch.Tensor, n: int) -> torch.Tensor:
        B = hidden.shape[0]
        w = self.w
        out = torch.empty(B, n, dtype=torch.int64, device=hidden.device)
        prev = hidden
        if self.cfg.scale_input:
            prev = spec_ops.spec_ln(prev, None, None, self.LN_EPS, 1.0 / math.sqrt(2.0))
        tok = tokens.to(torch.int64).contiguous()
        c = None
        for i in range(n):
            if self.lstm:
                gates = ops.linear(prev, w["projs.%d.weight" % min(i, 1)])
                c, prev = spec_ops.sum_lstm(gates, w["forget_emb.0.weight"], tok, self.alpha, c,
                                            w["cell_ln.0.weight"], w.get("cell_ln.0.bias"),
                                            w["state_ln.0.weight"], w.get("state_ln.0.bias"),
                                            self.LN_EPS)
                head = self._head("head.0.weight", B)
            else:
                k = self._idx("emb", i)
                proj = ops.linear(prev, w["proj.%d.weight" % self._idx("proj", i)])
                prev = spec_ops.mlp_spec_step(proj, w["emb.%d.weight" % k], tok, self.alpha,
                                              w["ln.%d.weight" % k], w.get("ln.%d.bias" % k),
                                              self.LN_EPS)
                head = self._head("head.%d.weight" % k, B)
            logits = ops.linear(prev, head)
            tp = getattr(self, "tp_comm", None)
            if tp is None:
                tok, _ = ops.argmax_sample(logits)
            else:
                ids, vals = ops.argmax_sample(logits, index_offset=self.tp_offset)
                tok = tp.argmax_exchange(ids, vals)
            tok = tok.clamp_(0, self.cfg.vocab_size - 1)
            out[:, i] = tok
        return out


def build_speculator(path_or_cfg, device="cuda", seed: int = 0) -> ArcticSpeculator:
    """A speculator from a checkpoint directory, or a random one from a config / preset dict."""
    if isinstance(path_or_cfg, SpeculatorConfig):
        spec = ArcticSpeculator(path_or_cfg, device)
        spec.init_random(seed)
        return spec
    if isinstance(path_or_cfg, dict):
        spec = ArcticSpeculator(SpeculatorConfig.from_dict(path_or_cfg), device)
        spec.init_random(seed)
        return spec
    cfg = SpeculatorConfig.from_pretrained(path_or_cfg)
    spec = ArcticSpeculator(cfg, device)
    spec.load_pretrained(path_or_cfg)
    return spec
