"""B200-native LLM / embedding inference engine with the capabilities of
Snowflake's ArcticInference: Ulysses sequence parallelism, shift parallelism,
SwiftKV, Arctic speculators with suffix decoding, the embedding service and the
replica server with live weight sync. PyTorch provides tensors, streams and CUDA
graphs; the hot ops are hand-written sm_100a kernels (``csrc/``)."""

__version__ = "0.1.0"

_LAZY = {
    "LLM": ("arcticinference_b200.engine.llm", "LLM"),
    "SamplingParams": ("arcticinference_b200.engine.sampling_params", "SamplingParams"),
    "EngineArgs": ("arcticinference_b200.config", "EngineArgs"),
    "RequestOutput": ("arcticinference_b200.engine.outputs", "RequestOutput"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib
        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(name)
