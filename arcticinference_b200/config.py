"""Configuration objects and the command-line flag system.

One set of dataclasses describes an engine; :class:`EngineArgs` is the flat,
CLI-facing view (``serve`` flags and ``LLM(...)`` keyword arguments) and
:meth:`EngineArgs.create_engine_config` validates it into an
:class:`EngineConfig`.

Parity notes (paths are the reference's): the Arctic flags and their defaults
come from arctic_inference/vllm/args.py:31-38,86-129; the parallel-size rules
from arctic_inference/vllm/config.py:30-46; the speculative-decoding fields,
defaults and batch-size caps from arctic_inference/vllm/config.py:50-170.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import logging
import os
from dataclasses import dataclass, field
from typing import Any, Optional

logger = logging.getLogger(__name__)


# --------------------------------------------------------------------------------------
# model
# --------------------------------------------------------------------------------------

SHIFT_PARALLEL_THRESHOLD = 128

@dataclass
class ModelConfig:
    """Architecture of a decoder (Llama, Mistral, Qwen2 and Qwen3 dense models, optionally
    SwiftKV for Llama) or encoder (BERT)."""

    architecture: str = "LlamaForCausalLM"
    model_type: str = "llama"
    hidden_size: int = 4096
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[dict] = None
    max_position_embeddings: int = 131072
    tie_word_embeddings: bool = False
    # SwiftKV: layers >= num_key_value_layers take K/V from a projection of the hidden
    # state after layer num_key_value_layers - 1 (None: plain Llama).
    num_key_value_layers: Optional[int] = None
    # Qwen3: RMSNorm over head_dim on every query and key head before RoPE
    qk_norm: bool = False
    # Qwen2: a bias on the query / key / value projections (none on o_proj or the MLP)
    qkv_bias: bool = False
    # attention window of the checkpoint (Mistral v0.1): contexts up to this length see every
    # earlier token, so they are served; longer ones are refused (no windowed attention kernel)
    sliding_window: Optional[int] = None
    # K/V heads of the checkpoint when ``num_key_value_heads`` was raised (see __post_init__)
    checkpoint_kv_heads: Optional[int] = None
    # encoder-only fields
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    pooling: str = "cls"  # cls | mean
    normalize: bool = True
    hidden_act: str = "silu"
    # weights
    dtype: str = "bfloat16"
    quantization: Optional[str] = None  # None | "fp8"
    fp8_block_size: int = 128
    # "channel": a scale per output feature, activations per token; "block": 128 x 128 blocks
    fp8_scheme: str = "channel"
    eos_token_id: Optional[int] = None
    # further end-of-sequence ids (a list in config.json or generation_config.json, e.g. the
    # end-of-turn token of instruction-tuned Llama 3): they end a request like EOS does
    extra_eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    name_or_path: str = ""

    def __post_init__(self):
        """The attention kernels pack the G = heads / kv_heads query heads of a K/V head into
        128-row tiles, so G must divide 128. A checkpoint with another ratio (Qwen2.5-7B: 7,
        14B / 32B: 5, 1.5B: 6) is served with each of its K/V heads stored r times, r the
        smallest divisor of G that leaves G / r a divisor of 128: the model is the same
        function, the KV cache is r times larger. ``num_key_value_heads`` is the number of
        heads stored; ``checkpoint_kv_heads`` keeps the checkpoint's."""
        hq, hkv = self.num_attention_heads, self.num_key_value_heads
        if self.is_encoder or hkv <= 0 or hq % hkv:
            return
        g = hq // hkv
        if 128 % g == 0:
            return
        r = next(r for r in range(2, g + 1) if g % r == 0 and 128 % (g // r) == 0)
        if self.checkpoint_kv_heads is None:
            self.checkpoint_kv_heads = hkv
        self.num_key_value_heads = hkv * r

    @property
    def kv_head_replication(self) -> int:
        return self.num_key_value_heads // (self.checkpoint_kv_heads or self.num_key_value_heads)

    @property
    def is_swiftkv(self) -> bool:
        return self.num_key_value_layers is not None and \
            self.num_key_value_layers < self.num_hidden_layers

    @property
    def is_encoder(self) -> bool:
        return self.model_type in ("bert",)

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim not in (64, 128):
            raise ValueError("head_dim must be 64 or 128 (tensor-memory attention tiles)")
        if self.quantization not in (None, "fp8"):
            raise ValueError("quantization must be None or 'fp8'")
        if self.fp8_scheme not in ("channel", "block"):
            raise ValueError("fp8_scheme must be 'channel' or 'block'")
        if (self.qk_norm or self.qkv_bias) and self.is_swiftkv:
            raise NotImplementedError("SwiftKV with per-head query / key norms or a QKV bias")
        if self.qkv_bias and self.quantization == "fp8" and self.fp8_scheme == "block":
            raise NotImplementedError("a QKV bias with block-scaled fp8 linears: use "
                                      "fp8_scheme='channel'")

    @classmethod
    def from_hf_dict(cls, d: dict, name_or_path: str = "") -> "ModelConfig":
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        mt = d.get("model_type", "llama")
        heads = d.get("num_attention_heads", 32)
        hidden = d.get("hidden_size", 4096)
        eos, extra_eos = d.get("eos_token_id"), ()
        if isinstance(eos, list):
            eos, extra_eos = (eos[0] if eos else None), tuple(int(t) for t in eos[1:])
        if mt not in DECODER_MODEL_TYPES and mt != "bert":
            raise NotImplementedError("model_type %r (supported: %s, bert)" %
                                      (mt, ", ".join(DECODER_MODEL_TYPES)))
        if d.get("attention_bias") or d.get("mlp_bias"):
            # (Llama's attention_bias also puts a bias on o_proj; Qwen2's QKV-only bias is
            # part of its architecture and has no flag)
            raise NotImplementedError("linear layers with bias (attention_bias / mlp_bias)")
        window = d.get("sliding_window") if d.get("use_sliding_window", True) else None
        # transformers >= 5 writes one ``rope_parameters`` dict (theta, type and the scaling
        # fields together); older checkpoints have ``rope_theta`` beside ``rope_scaling``
        rope = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope.get("rope_theta", 10000.0))
        scaling = d.get("rope_scaling")
        if scaling is None and rope.get("rope_type", rope.get("type", "default")) != "default":
            scaling = {k: v for k, v in rope.items() if k != "rope_theta"}
        cfg = cls(
            architecture=archs[0], model_type=mt, hidden_size=hidden,
            num_hidden_layers=d.get("num_hidden_layers", 32), num_attention_heads=heads,
            num_key_value_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or hidden // heads,
            intermediate_size=d.get("intermediate_size", 4 * hidden),
            vocab_size=d.get("vocab_size", 32000),
            rms_norm_eps=d.get("rms_norm_eps", 1e-5),
            rope_theta=theta, rope_scaling=scaling,
            max_position_embeddings=d.get("max_position_embeddings", 4096),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            num_key_value_layers=d.get("num_key_value_layers"),
            qk_norm=(mt == "qwen3"), qkv_bias=(mt == "qwen2"), sliding_window=window,
            type_vocab_size=d.get("type_vocab_size", 2),
            layer_norm_eps=d.get("layer_norm_eps", 1e-12),
            hidden_act=d.get("hidden_act", "silu"),
            eos_token_id=eos, extra_eos_token_ids=extra_eos, bos_token_id=d.get("bos_token_id"),
            name_or_path=name_or_path)
        q = d.get("quantization_config")
        if q and q.get("quant_method") in ("fp8", "compressed-tensors"):
            cfg.quantization = "fp8"
            wbs = q.get("weight_block_size")
            if wbs:
                cfg.fp8_block_size = int(wbs[0])
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        if path in PRESETS:
            return dataclasses.replace(PRESETS[path], name_or_path=path)
        with open(os.path.join(path, "config.json")) as f:
            cfg = cls.from_hf_dict(json.load(f), path)
        gen = os.path.join(path, "generation_config.json")
        if os.path.exists(gen):
            with open(gen) as f:
                ids = json.load(f).get("eos_token_id")
            ids = [] if ids is None else ([int(t) for t in ids] if isinstance(ids, list) else [int(ids)])
            if cfg.eos_token_id is None and ids:
                cfg.eos_token_id = ids[0]
            known = {cfg.eos_token_id, *cfg.extra_eos_token_ids}
            cfg.extra_eos_token_ids += tuple(t for t in dict.fromkeys(ids) if t not in known)
        return cfg


# decoder families the Llama code path serves: Mistral is Llama under another name once its
# sliding window is off; Qwen2 adds a bias on the QKV projection; Qwen3 (dense) adds the
# per-head query / key norms and a head_dim that is not hidden_size / heads
DECODER_MODEL_TYPES = ("llama", "llama_swiftkv", "mistral", "qwen2", "qwen3")


def _llama(layers, hidden, heads, kv, inter, **kw) -> ModelConfig:
    return ModelConfig(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                       num_key_value_heads=kv, head_dim=128, intermediate_size=inter, **kw)


_LLAMA3_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                   "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}

# Synthetic (random-weight) presets for the architectures the benchmarks name.
PRESETS: dict[str, ModelConfig] = {
    "llama-3.1-8b": _llama(32, 4096, 32, 8, 14336, rope_scaling=dict(_LLAMA3_SCALING)),
    "llama-3.1-8b-swiftkv": _llama(32, 4096, 32, 8, 14336, rope_scaling=dict(_LLAMA3_SCALING),
                                   num_key_value_layers=16, model_type="llama_swiftkv",
                                   architecture="LlamaSwiftKVForCausalLM"),
    "llama-3.3-70b": _llama(80, 8192, 64, 8, 28672, rope_scaling=dict(_LLAMA3_SCALING)),
    "llama-3.3-70b-swiftkv": _llama(80, 8192, 64, 8, 28672, rope_scaling=dict(_LLAMA3_SCALING),
                                    num_key_value_layers=40, model_type="llama_swiftkv",
                                    architecture="LlamaSwiftKVForCausalLM"),
    "llama-tiny": ModelConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                              num_key_value_heads=2, head_dim=64, intermediate_size=512,
                              vocab_size=1024, max_position_embeddings=4096, rope_theta=10000.0),
    "llama-tiny-swiftkv": ModelConfig(hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                                      num_key_value_heads=2, head_dim=64, intermediate_size=512,
                                      vocab_size=1024, max_position_embeddings=4096,
                                      rope_theta=10000.0, num_key_value_layers=2,
                                      model_type="llama_swiftkv",
                                      architecture="LlamaSwiftKVForCausalLM"),
    "mistral-7b": _llama(32, 4096, 32, 8, 14336, architecture="MistralForCausalLM",
                         model_type="mistral", vocab_size=32768, rope_theta=1000000.0,
                         max_position_embeddings=32768),
    "qwen2.5-7b": _llama(28, 3584, 28, 4, 18944, architecture="Qwen2ForCausalLM",
                         model_type="qwen2", qkv_bias=True, vocab_size=152064,
                         rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=32768),
    # the reasoning model of the Dynasor examples (a Qwen2 architecture)
    "deepseek-r1-distill-qwen-1.5b": ModelConfig(
        architecture="Qwen2ForCausalLM", model_type="qwen2", qkv_bias=True, hidden_size=1536,
        num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
        intermediate_size=8960, vocab_size=151936, rope_theta=10000.0, rms_norm_eps=1e-6,
        max_position_embeddings=131072),
    "qwen2-tiny": ModelConfig(architecture="Qwen2ForCausalLM", model_type="qwen2", qkv_bias=True,
                              hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                              num_key_value_heads=2, head_dim=64, intermediate_size=512,
                              vocab_size=1024, max_position_embeddings=4096, rope_theta=10000.0,
                              rms_norm_eps=1e-6),
    "qwen3-8b": _llama(36, 4096, 32, 8, 12288, architecture="Qwen3ForCausalLM",
                       model_type="qwen3", qk_norm=True, vocab_size=151936, rope_theta=1000000.0,
                       rms_norm_eps=1e-6, max_position_embeddings=40960),
    "qwen3-32b": _llama(64, 5120, 64, 8, 25600, architecture="Qwen3ForCausalLM",
                        model_type="qwen3", qk_norm=True, vocab_size=151936, rope_theta=1000000.0,
                        rms_norm_eps=1e-6, max_position_embeddings=40960),
    "qwen3-tiny": ModelConfig(architecture="Qwen3ForCausalLM", model_type="qwen3", qk_norm=True,
                              hidden_size=256, num_hidden_layers=2, num_attention_heads=8,
                              num_key_value_heads=2, head_dim=64, intermediate_size=512,
                              vocab_size=1024, max_position_embeddings=4096, rope_theta=10000.0,
                              rms_norm_eps=1e-6),
    "llama-small": ModelConfig(hidden_size=1024, num_hidden_layers=4, num_attention_heads=8,
                               num_key_value_heads=8, head_dim=128, intermediate_size=2816,
                               vocab_size=32000, max_position_embeddings=8192),
    "bert-base": ModelConfig(architecture="BertModel", model_type="bert", hidden_size=768,
                             num_hidden_layers=12, num_attention_heads=12, num_key_value_heads=12,
                             head_dim=64, intermediate_size=3072, vocab_size=30522,
                             max_position_embeddings=512, hidden_act="gelu"),
    "bert-tiny": ModelConfig(architecture="BertModel", model_type="bert", hidden_size=128,
                             num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2,
                             head_dim=64, intermediate_size=256, vocab_size=1000,
                             max_position_embeddings=512, hidden_act="gelu"),
}


# --------------------------------------------------------------------------------------
# parallelism
# --------------------------------------------------------------------------------------
@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    ulysses_sequence_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_shift_parallel: bool = False
    # steps with at most this many tokens run tensor-parallel. The reference's default is 512;
    # here 128 (one 128-token tile per linear, the shape the decode GEMMs are built for):
    # measured on 2 GPUs, 256-token decode steps serve 5 % more tokens/s sequence-parallel
    shift_parallel_threshold: int = SHIFT_PARALLEL_THRESHOLD
    enable_expert_parallel: bool = False
    # "fused": own NVLink kernels; "nccl": library collectives (kept for A/B runs)
    comm_backend: str = "fused"

    def __post_init__(self):
        if self.enable_shift_parallel and self.ulysses_sequence_parallel_size == 1:
            raise ValueError("ulysses_sequence_parallel_size must be > 1 "
                             "when enable_shift_parallel is True.")
        for name in ("tensor_parallel_size", "ulysses_sequence_parallel_size",
                     "pipeline_parallel_size", "data_parallel_size"):
            if getattr(self, name) < 1:
                raise ValueError("%s must be >= 1" % name)
        if self.comm_backend not in ("fused", "nccl"):
            raise ValueError("comm_backend must be 'fused' or 'nccl'")

    @property
    def world_size(self) -> int:
        """Ranks of one engine replica: PP x SP x TP (data-parallel replicas are separate)."""
        return (self.pipeline_parallel_size * self.tensor_parallel_size *
                self.ulysses_sequence_parallel_size)

    @property
    def sp(self) -> int:
        return self.ulysses_sequence_parallel_size

    @property
    def tp(self) -> int:
        return self.tensor_parallel_size


# --------------------------------------------------------------------------------------
# speculative decoding
# --------------------------------------------------------------------------------------
@dataclass
class SpeculativeConfig:
    method: Optional[str] = None  # arctic | mlp_speculator | suffix
    model: Optional[str] = None
    num_speculative_tokens: Optional[int] = None
    disable_by_batch_size: Optional[int] = None
    hard_disable_by_batch_size: Optional[int] = None
    enable_suffix_decoding: bool = False
    suffix_cache_max_depth: int = 64
    suffix_speculative_tokens: int = 0
    suffix_cache_max_requests: int = 100000
    suffix_max_spec_factor: float = 1.0
    suffix_max_spec_offset: float = 0.0
    suffix_min_token_prob: float = 0.1
    draft_tensor_parallel_size: Optional[int] = None
    quantization: Optional[str] = None     # "fp8": block-scaled fp8 projections and LM heads of the drafter

    def __post_init__(self):
        if self.quantization not in (None, "fp8"):
            raise ValueError("speculator quantization must be None or 'fp8'")
        if self.method not in (None, "arctic", "mlp_speculator", "suffix"):
            raise ValueError("unknown speculative method %r" % (self.method,))
        arctic = self.method in ("arctic", "mlp_speculator")
        suffix_only = self.method == "suffix" or (self.method is None and
                                                  self.enable_suffix_decoding)
        hybrid = self.method == "arctic" and self.enable_suffix_decoding
        if (suffix_only or arctic) and self.disable_by_batch_size is None:
            self.disable_by_batch_size = 64
        if (self.hard_disable_by_batch_size is not None and
                self.disable_by_batch_size is not None and
                self.hard_disable_by_batch_size <= self.disable_by_batch_size):
            logger.warning("hard_disable_by_batch_size=%d <= disable_by_batch_size=%d: "
                           "the first-N cap never applies", self.hard_disable_by_batch_size,
                           self.disable_by_batch_size)
        if hybrid:
            self.suffix_speculative_tokens = self.suffix_cache_max_depth
        if suffix_only:
            self.method = "suffix"
            self.enable_suffix_decoding = True
            if self.suffix_speculative_tokens > 0:
                self.num_speculative_tokens = self.suffix_speculative_tokens
            elif self.num_speculative_tokens is None:
                self.num_speculative_tokens = 16
        elif arctic:
            if self.model is None:
                raise ValueError("speculative method %r needs a draft 'model'" % self.method)
            if not self.num_speculative_tokens:
                self.num_speculative_tokens = None  # filled from the draft model's n_predict
        if self.num_speculative_tokens is not None and self.num_speculative_tokens < 0:
            raise ValueError("num_speculative_tokens must be >= 0")

    @property
    def uses_arctic(self) -> bool:
        return self.method in ("arctic", "mlp_speculator")

    @property
    def uses_suffix(self) -> bool:
        return self.enable_suffix_decoding

    @property
    def max_draft_tokens(self) -> int:
        """Widest draft any request can carry into a verification step."""
        return max(self.num_speculative_tokens or 0, self.suffix_speculative_tokens or 0)

    def effective_draft_limit(self, batch_size: int) -> int:
        """How many requests of a running batch may draft this step: 0 once the batch
        reaches the hard cap, the first ``disable_by_batch_size`` above the soft cap,
        everyone otherwise."""
        if (self.hard_disable_by_batch_size is not None and
                batch_size >= self.hard_disable_by_batch_size):
            return 0
        if self.disable_by_batch_size is not None and batch_size > self.disable_by_batch_size:
            return self.disable_by_batch_size
        return batch_size

    @classmethod
    def from_json(cls, value) -> Optional["SpeculativeConfig"]:
        if value is None:
            return None
        if isinstance(value, cls):
            return value
        if isinstance(value, str):
            value = json.loads(value)
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = set(value) - known
        if unknown:
            raise ValueError("unknown speculative-config keys: %s" % sorted(unknown))
        return cls(**value)


# --------------------------------------------------------------------------------------
# cache / scheduler / forest cascade attention
# --------------------------------------------------------------------------------------
# cache element types the attention kernels can read (the cache writers also produce nvfp4)
SUPPORTED_KV_CACHE_DTYPES = ("auto", "bfloat16")


@dataclass
class CacheConfig:
    block_size: int = 64
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks: Optional[int] = None  # None: sized from free memory
    kv_cache_dtype: str = "auto"  # auto (= model dtype) | fp8 | nvfp4
    enable_prefix_caching: bool = True

    def __post_init__(self):
        if self.block_size not in (16, 32, 64, 128):
            raise ValueError("block_size must be 16, 32, 64 or 128")
        if self.kv_cache_dtype not in ("auto", "bfloat16", "fp8", "nvfp4"):
            raise ValueError("unsupported kv_cache_dtype %r" % self.kv_cache_dtype)


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 256
    max_model_len: int = 8192
    enable_chunked_prefill: bool = True
    async_scheduling: bool = False


@dataclass
class ForestCascadeConfig:
    """Gates of forest cascade attention (shared-prefix grouping of decode batches);
    defaults as in arctic_inference/vllm/attention/flash_attn_forest_cascade.py:304-319."""
    enabled: bool = False
    max_query_len: int = 16
    min_batch_size: int = 8
    min_group_size: int = 2
    min_additional_prefix_blocks: int = 1
    min_non_singleton_fraction: float = 0.25
    max_non_singleton_groups: int = 256

    @classmethod
    def from_json(cls, value) -> "ForestCascadeConfig":
        if value is None:
            return cls(enabled=False)
        if isinstance(value, str):
            value = json.loads(value)
        known = {f.name for f in dataclasses.fields(cls)} - {"enabled"}
        unknown = set(value) - known
        if unknown:
            raise ValueError("unknown forest-cascade-attn keys: %s" % sorted(unknown))
        return cls(enabled=True, **value)


@dataclass
class EngineConfig:
    model: ModelConfig
    parallel: ParallelConfig
    cache: CacheConfig
    scheduler: SchedulerConfig
    speculative: Optional[SpeculativeConfig] = None
    forest_cascade: ForestCascadeConfig = field(default_factory=ForestCascadeConfig)
    fp32_lm_head: bool = False
    enforce_eager: bool = False
    enable_sleep_mode: bool = False
    seed: int = 0
    load_format: str = "auto"  # auto | dummy (random weights)
    tokenizer: Optional[str] = None
    served_model_name: Optional[str] = None

    def validate(self) -> None:
        m, p = self.model, self.parallel
        m.validate()
        ways = p.tp * p.sp
        if m.num_attention_heads % ways:
            raise ValueError("num_attention_heads (%d) must be divisible by TP*SP (%d)" %
                             (m.num_attention_heads, ways))
        if m.num_key_value_heads % p.tp and p.tp % m.num_key_value_heads:
            raise ValueError("num_key_value_heads and tensor_parallel_size must divide evenly")
        if m.is_swiftkv and p.pipeline_parallel_size > 1:
            raise ValueError("SwiftKV models do not support pipeline parallelism")
        if m.sliding_window is not None and self.scheduler.max_model_len > m.sliding_window:
            raise NotImplementedError(
                "sliding-window attention: this checkpoint attends to the last %d tokens only; "
                "contexts up to that length are served (max_model_len=%d asks for more)"
                % (m.sliding_window, self.scheduler.max_model_len))
        if not m.is_encoder:
            per_rank = (m.num_attention_heads // ways) // max(1, m.num_key_value_heads // ways)
            if per_rank < 1 or 128 % per_rank:
                raise NotImplementedError(
                    "%d query heads per K/V head on a rank (TP*SP = %d): the attention kernels "
                    "need a divisor of 128" % (per_rank, ways))
        # Options this engine parses for command-line compatibility but cannot honour are
        # refused here rather than ignored.
        if p.pipeline_parallel_size > 1:
            # whole-model stages (parallel/pipeline.py): one rank per stage, nothing sharded
            # inside a stage, no drafting (the drafter lives with the last stage's hidden states)
            if p.tp * p.sp > 1:
                raise NotImplementedError(
                    "pipeline_parallel_size > 1 together with tensor or sequence parallelism: "
                    "pipeline stages are whole-model stages here (TP = SP = 1)")
            if self.speculative is not None:
                raise NotImplementedError("speculative decoding with pipeline parallelism")
            if p.pipeline_parallel_size > m.num_hidden_layers:
                raise ValueError("more pipeline stages than decoder layers")
        if p.data_parallel_size > 1:
            raise NotImplementedError(
                "data_parallel_size > 1: replicas are separate engines here; start one server "
                "per replica, or use the replica pool (python -m arcticinference_b200.server.cli), "
                "which routes requests over them")
        if p.enable_expert_parallel:
            raise NotImplementedError("enable_expert_parallel: no mixture-of-experts model is "
                                      "implemented, so there is nothing to shard by expert")
        if self.cache.kv_cache_dtype not in SUPPORTED_KV_CACHE_DTYPES:
            raise NotImplementedError(
                "kv_cache_dtype=%r: the attention kernels read %s caches only" %
                (self.cache.kv_cache_dtype, " / ".join(SUPPORTED_KV_CACHE_DTYPES)))
        if self.speculative is not None and self.speculative.uses_suffix and \
                self.speculative.method not in ("arctic", "suffix"):
            raise ValueError("suffix decoding is only available with the arctic or suffix methods")
        if self.scheduler.max_num_batched_tokens < p.sp:
            raise ValueError("max_num_batched_tokens must be >= the sequence-parallel size")

    @property
    def kv_replication(self) -> int:
        """How many ranks hold a copy of each KV head (>1 when Hkv < TP*SP)."""
        ways = self.parallel.tp * self.parallel.sp
        return max(1, ways // self.model.num_key_value_heads)


# --------------------------------------------------------------------------------------
# flat CLI / keyword view
# --------------------------------------------------------------------------------------
def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").lower() in ("1", "true", "on", "yes")


@dataclass
class EngineArgs:
    model: str = "llama-tiny"
    tokenizer: Optional[str] = None
    served_model_name: Optional[str] = None
    dtype: str = "bfloat16"
    quantization: Optional[str] = None
    fp8_scheme: Optional[str] = None
    load_format: str = "auto"
    seed: int = 0
    max_model_len: Optional[int] = None
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    # Arctic flags
    ulysses_sequence_parallel_size: int = 1
    enable_shift_parallel: bool = False
    shift_parallel_threshold: int = SHIFT_PARALLEL_THRESHOLD
    forest_cascade_attn_configs: Optional[Any] = None
    fp32_lm_head: bool = False
    speculative_config: Optional[Any] = None
    # engine
    block_size: int = 64
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks_override: Optional[int] = None
    kv_cache_dtype: str = "auto"
    enable_prefix_caching: bool = True
    max_num_batched_tokens: Optional[int] = None
    max_num_seqs: int = 256
    enable_chunked_prefill: bool = True
    async_scheduling: bool = True
    enforce_eager: bool = False
    enable_sleep_mode: bool = False
    comm_backend: str = "fused"
    distributed_executor_backend: Optional[str] = None
    hf_overrides: Optional[dict] = None

    def __post_init__(self):
        # Sequence parallelism always runs one process per GPU (arctic_inference/vllm/args.py:71-73).
        if self.ulysses_sequence_parallel_size > 1:
            self.distributed_executor_backend = "mp"
        if self.distributed_executor_backend not in (None, "mp", "external_launcher"):
            # one process per GPU under torch.distributed is the only executor there is
            raise NotImplementedError("distributed_executor_backend=%r (ranks are processes "
                                      "started by serve or torch.distributed.run)"
                                      % self.distributed_executor_backend)
        if _env_flag("ARCTIC_FP32_LM_HEAD"):
            self.fp32_lm_head = True

    # ---- CLI ---------------------------------------------------------------------------
    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        g = parser.add_argument_group("model")
        g.add_argument("--tokenizer", type=str, default=None)
        g.add_argument("--served-model-name", type=str, default=None)
        g.add_argument("--dtype", type=str, default="bfloat16")
        g.add_argument("--quantization", "-q", type=str, default=None, choices=[None, "fp8"])
        g.add_argument("--fp8-scheme", type=str, default=None, choices=[None, "channel", "block"],
                       help="fp8 scale layout: one scale per output feature with per-token "
                            "activation scales (default), or 128 x 128 blocks")
        g.add_argument("--load-format", type=str, default="auto", choices=["auto", "dummy"])
        g.add_argument("--seed", type=int, default=0)
        g.add_argument("--max-model-len", type=int, default=None)
        g.add_argument("--hf-overrides", type=json.loads, default=None)
        g = parser.add_argument_group("parallelism")
        g.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
        g.add_argument("--pipeline-parallel-size", "-pp", type=int, default=1)
        g.add_argument("--data-parallel-size", "-dp", type=int, default=1)
        g.add_argument("--enable-expert-parallel", action="store_true")
        g.add_argument("--ulysses-sequence-parallel-size", type=int, default=1,
                       help="Number of Ulysses sequence parallel replicas")
        g.add_argument("--enable-shift-parallel", action="store_true",
                       help="Switch between sequence parallelism and full tensor parallelism "
                            "per step, by batch size")
        g.add_argument("--shift-parallel-threshold", type=int, default=SHIFT_PARALLEL_THRESHOLD,
                       help="Steps with at most this many tokens run in tensor-parallel mode")
        g.add_argument("--comm-backend", type=str, default="fused", choices=["fused", "nccl"])
        g.add_argument("--distributed-executor-backend", type=str, default=None)
        g = parser.add_argument_group("arctic")
        g.add_argument("--forest-cascade-attn-configs", type=str, default=None,
                       help="JSON object of forest cascade attention knobs; '{}' enables defaults")
        g.add_argument("--fp32-lm-head", action="store_true",
                       help="Compute the LM head in fp32")
        g.add_argument("--speculative-config", type=str, default=None,
                       help="JSON: method arctic|mlp_speculator|suffix, model, "
                            "num_speculative_tokens, enable_suffix_decoding, ...")
        g = parser.add_argument_group("engine")
        g.add_argument("--block-size", type=int, default=64)
        g.add_argument("--gpu-memory-utilization", type=float, default=0.9)
        g.add_argument("--num-gpu-blocks-override", type=int, default=None)
        g.add_argument("--kv-cache-dtype", type=str, default="auto")
        g.add_argument("--enable-prefix-caching", dest="enable_prefix_caching",
                       action="store_true", default=True)
        g.add_argument("--no-enable-prefix-caching", dest="enable_prefix_caching",
                       action="store_false")
        g.add_argument("--max-num-batched-tokens", type=int, default=None)
        g.add_argument("--max-num-seqs", type=int, default=256)
        g.add_argument("--enable-chunked-prefill", dest="enable_chunked_prefill",
                       action="store_true", default=True)
        g.add_argument("--no-enable-chunked-prefill", dest="enable_chunked_prefill",
                       action="store_false")
        g.add_argument("--async-scheduling", dest="async_scheduling", action="store_true", default=True,
                       help="queue the next decode step before the previous step's tokens are read")
        g.add_argument("--no-async-scheduling", dest="async_scheduling", action="store_false")
        g.add_argument("--enforce-eager", action="store_true")
        g.add_argument("--enable-sleep-mode", action="store_true")
        return parser

    @classmethod
    def from_cli_args(cls, ns: argparse.Namespace) -> "EngineArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in vars(ns).items() if k in names})

    # ---- validation into an EngineConfig -------------------------------------------------
    def create_engine_config(self) -> EngineConfig:
        model = ModelConfig.from_pretrained(self.model)
        if self.hf_overrides:
            model = dataclasses.replace(model, **self.hf_overrides)
        if self.quantization is not None:
            model.quantization = self.quantization
        if self.fp8_scheme is not None:
            model.fp8_scheme = self.fp8_scheme
        if self.dtype not in ("auto", "bfloat16", "bf16"):
            raise NotImplementedError("dtype=%r: weights, activations and the KV cache are "
                                      "bfloat16 (the kernels accumulate in fp32)" % self.dtype)
        model.dtype = "bfloat16"
        max_len = self.max_model_len or min(model.max_position_embeddings, 8192,
                                            model.sliding_window or 8192)
        parallel = ParallelConfig(
            tensor_parallel_size=self.tensor_parallel_size,
            ulysses_sequence_parallel_size=self.ulysses_sequence_parallel_size,
            pipeline_parallel_size=self.pipeline_parallel_size,
            data_parallel_size=self.data_parallel_size,
            enable_shift_parallel=self.enable_shift_parallel,
            shift_parallel_threshold=self.shift_parallel_threshold,
            enable_expert_parallel=self.enable_expert_parallel,
            comm_backend=self.comm_backend)
        cache = CacheConfig(block_size=self.block_size,
                            gpu_memory_utilization=self.gpu_memory_utilization,
                            num_gpu_blocks=self.num_gpu_blocks_override,
                            kv_cache_dtype=self.kv_cache_dtype,
                            enable_prefix_caching=self.enable_prefix_caching)
        sched = SchedulerConfig(
            max_num_batched_tokens=self.max_num_batched_tokens or max(8192, 0),
            max_num_seqs=self.max_num_seqs, max_model_len=max_len,
            enable_chunked_prefill=self.enable_chunked_prefill,
            async_scheduling=self.async_scheduling)
        spec = SpeculativeConfig.from_json(self.speculative_config)
        cfg = EngineConfig(
            model=model, parallel=parallel, cache=cache, scheduler=sched, speculative=spec,
            forest_cascade=ForestCascadeConfig.from_json(self.forest_cascade_attn_configs),
            fp32_lm_head=self.fp32_lm_head, enforce_eager=self.enforce_eager,
            enable_sleep_mode=self.enable_sleep_mode, seed=self.seed,
            load_format="dummy" if self.model in PRESETS else self.load_format,
            tokenizer=self.tokenizer, served_model_name=self.served_model_name or self.model)
        cfg.validate()
        return cfg
