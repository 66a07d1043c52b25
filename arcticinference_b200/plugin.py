"""Model registry and start-up checks.

The reference is loaded by vLLM as a plugin that registers its model classes and applies its
patches (arctic_inference/vllm/plugin.py:25-46, arctic_inference/vllm/patches.py:313-370). Here
there is nothing to patch; what remains is the registry that maps Hugging Face architecture
names to this engine's model classes, and the platform check.
"""

from __future__ import annotations

import logging
from typing import Callable

from . import envs

logger = logging.getLogger(__name__)

_MODEL_REGISTRY: dict[str, Callable] = {}
_CONFIG_REGISTRY: dict[str, str] = {}


def register_model(architecture: str, factory: Callable) -> None:
    _MODEL_REGISTRY[architecture] = factory


def register_config(model_type: str, description: str) -> None:
    _CONFIG_REGISTRY[model_type] = description


def resolve_model(architecture: str) -> Callable:
    _ensure_registered()
    if architecture not in _MODEL_REGISTRY:
        raise KeyError("unsupported architecture %r; known: %s" %
                       (architecture, sorted(_MODEL_REGISTRY)))
    return _MODEL_REGISTRY[architecture]


def supported_architectures() -> list[str]:
    _ensure_registered()
    return sorted(_MODEL_REGISTRY)


def _ensure_registered() -> None:
    if _MODEL_REGISTRY:
        return

    def _llama(*a, **k):
        from .models.llama import LlamaForCausalLM
        return LlamaForCausalLM(*a, **k)

    def _speculator(*a, **k):
        from .models.speculator import build_speculator
        return build_speculator(*a, **k)

    def _bert(*a, **k):
        from .models.bert import BertEncoder
        return BertEncoder(*a, **k)

    register_config("llama_swiftkv", "Llama with SwiftKV (num_key_value_layers)")
    for arch in ("LlamaForCausalLM", "LlamaSwiftKVForCausalLM", "MistralForCausalLM",
                 "Qwen2ForCausalLM", "Qwen3ForCausalLM"):
        register_model(arch, _llama)
    for arch in ("ArcticMLPSpeculatorPreTrainedModel", "ArcticLSTMSpeculatorPreTrainedModel",
                 "MLPVariantSpeculatorPreTrainedModel", "MLPSpeculatorPreTrainedModel"):
        register_model(arch, _speculator)
    for arch in ("BertModel", "BertForMaskedLM"):
        register_model(arch, _bert)


def check_platform() -> None:
    """The kernels are built for sm_100a only."""
    if envs.ARCTIC_INFERENCE_SKIP_PLATFORM_CHECK:
        return
    import torch
    if not torch.cuda.is_available():
        return
    major, minor = torch.cuda.get_device_capability()
    if (major, minor) != (10, 0):
        raise RuntimeError("arcticinference_b200 kernels target sm_100a (B200); found sm_%d%d. "
                           "Set ARCTIC_INFERENCE_SKIP_PLATFORM_CHECK=1 to continue anyway." %
                           (major, minor))


def arctic_inference_plugin() -> None:
    """Entry point with the reference's name: registers models when the features are enabled."""
    if not envs.arctic_inference_effective_enabled():
        return
    check_platform()
    _ensure_registered()
