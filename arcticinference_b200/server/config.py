"""Server-side model configuration and the registry of tuned per-GPU settings.

``ServerModelConfig`` carries the engine arguments of one model plus two serving toggles
(``use_fca``: forest cascade attention, ``spec_model``: Arctic speculator path) that are
translated into real engine arguments, as the reference does for its vLLM engine
(arctic_inference/server/config.py:26-81). The registry is keyed by GPU type and by the model's
base name with quantisation suffixes removed (:10-13, :83-122); entries here are the dense
Llama-family models this framework serves on B200.
"""

from __future__ import annotations

import os
import re
from enum import Enum
from typing import Any, Optional

from pydantic import BaseModel, Field


_QUANT_SUFFIX = re.compile(r"-(FP8|NVFP4|FP4)(-dynamic)?$", re.IGNORECASE)


def normalize_model_name(name: str) -> str:
    return _QUANT_SUFFIX.sub("", name.rstrip("/").split("/")[-1])


class GPUType(str, Enum):
    H200 = "H200"
    B200 = "B200"


class ServerModelConfig(BaseModel):
    model: str = Field(description="preset name or local checkpoint directory")
    tensor_parallel_size: int = 1
    ulysses_sequence_parallel_size: int = 1
    enable_shift_parallel: bool = False
    shift_parallel_threshold: Optional[int] = None      # None: the engine's default
    max_model_len: int = 32768
    max_num_seqs: int = 1024
    max_num_batched_tokens: Optional[int] = None
    gpu_memory_utilization: float = 0.9
    quantization: Optional[str] = None
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = True
    kv_cache_dtype: Optional[str] = None
    enable_sleep_mode: bool = True
    enable_expert_parallel: bool = False    # passed on; the engine refuses it (no MoE model)
    # fields of the reference's schema that need nothing here: no checkpoint code is ever
    # executed, and replicas are processes pinned to whole GPUs, not Ray actors
    trust_remote_code: bool = True
    ray_num_gpus: Optional[float] = None
    use_fca: bool = False
    spec_model: str = ""
    extra_engine_kwargs: dict[str, Any] = Field(default_factory=dict)
    extra_env: dict[str, str] = Field(default_factory=dict)
    gpus_per_replica: Optional[int] = None

    @property
    def world_size(self) -> int:
        return self.tensor_parallel_size * self.ulysses_sequence_parallel_size

    def to_engine_kwargs(self) -> dict[str, Any]:
        skip = {"use_fca", "spec_model", "extra_engine_kwargs", "extra_env", "gpus_per_replica",
                "trust_remote_code", "ray_num_gpus"}
        kw = {k: v for k, v in self.model_dump().items() if v is not None and k not in skip}
        kw.update(self.extra_engine_kwargs)
        # the Arctic features are part of this engine, so they are on unless the launcher's or
        # the worker's environment switches them off explicitly
        val = self.extra_env.get("ARCTIC_INFERENCE_ENABLED", os.environ.get("ARCTIC_INFERENCE_ENABLED"))
        enabled = val is None or str(val).lower() not in ("0", "false", "off", "no", "")
        if enabled:
            if self.use_fca:
                kw.setdefault("forest_cascade_attn_configs", "{}")
            if self.spec_model:
                kw.setdefault("speculative_config", {"method": "arctic", "model": self.spec_model,
                                                     "num_speculative_tokens": 3})
        else:
            kw.pop("forest_cascade_attn_configs", None)
            kw.pop("speculative_config", None)
        return kw

    @classmethod
    def from_registry(cls, name: str, gpu_type: GPUType = GPUType.B200,
                      max_model_len: int = 32768) -> "ServerModelConfig":
        key = normalize_model_name(name)
        table = MODEL_CONFIGS.get(GPUType(gpu_type), {})
        if key not in table:
            raise ValueError("no tuned config for model=%r on gpu=%s" % (key, GPUType(gpu_type).value))
        return cls(max_model_len=max_model_len, **table[key])


# backwards-friendly alias: the reference's REST schema calls this ``ModelConfig``
ModelConfig = ServerModelConfig

MODEL_CONFIGS: dict[GPUType, dict[str, dict[str, Any]]] = {
    GPUType.B200: {
        "Llama-3.1-8B-Instruct": dict(model="llama-3.1-8b", quantization="fp8"),
        "Llama-3.1-8B-Instruct-SwiftKV": dict(model="llama-3.1-8b-swiftkv", quantization="fp8",
                                              use_fca=False),
        "Llama-3.3-70B-Instruct": dict(model="llama-3.3-70b", quantization="fp8",
                                       ulysses_sequence_parallel_size=8, enable_shift_parallel=True),
        "Llama-3.1-70B-Instruct": dict(model="llama-3.3-70b", quantization="fp8",
                                       ulysses_sequence_parallel_size=4, enable_shift_parallel=True),
        "Qwen3-8B": dict(model="qwen3-8b", quantization="fp8"),
        "Qwen3-32B": dict(model="qwen3-32b", quantization="fp8",
                          ulysses_sequence_parallel_size=4, enable_shift_parallel=True),
        "Mistral-7B-Instruct": dict(model="mistral-7b", quantization="fp8"),
    },
    GPUType.H200: {},
}
