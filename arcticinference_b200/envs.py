"""Environment switches, read lazily at attribute access (module ``__getattr__``), with the
names the reference uses (arctic_inference/envs.py:40-57 and the knobs scattered over
server/replica_pool.py:57-62, server/scheduler.py:21, weight_sync/receiver.py:185)."""

from __future__ import annotations

import os
from typing import Any, Callable, Optional


def _flag(name: str, default: str = "0") -> Callable[[], bool]:
    return lambda: os.getenv(name, default).lower() in ("1", "true", "on", "yes")


environment_variables: dict[str, Callable[[], Any]] = {
    "ARCTIC_INFERENCE_ENABLED": _flag("ARCTIC_INFERENCE_ENABLED"),
    "ARCTIC_INFERENCE_SKIP_PLATFORM_CHECK": _flag("ARCTIC_INFERENCE_SKIP_PLATFORM_CHECK"),
    "ARCTIC_INFERENCE_SKIP_SPEC_MODEL_CHECK": _flag("ARCTIC_INFERENCE_SKIP_SPEC_MODEL_CHECK"),
    "ARCTIC_INFERENCE_SKIP_VERSION_CHECK": _flag("ARCTIC_INFERENCE_SKIP_VERSION_CHECK"),
    "ARCTIC_FP32_LM_HEAD": _flag("ARCTIC_FP32_LM_HEAD"),
    "ARCTIC_PREFIX_ROUTING_DISABLED": _flag("ARCTIC_PREFIX_ROUTING_DISABLED"),
    "ARCTIC_LOG_AFFINITY": _flag("ARCTIC_LOG_AFFINITY"),
    "ARCTIC_WEIGHT_SYNC_STRICT_NAMES": _flag("ARCTIC_WEIGHT_SYNC_STRICT_NAMES", "1"),
    "ARCTIC_B200_NO_AUTOBUILD": _flag("ARCTIC_B200_NO_AUTOBUILD"),
    "ARCTIC_B200_COMM_BACKEND": lambda: os.getenv("ARCTIC_B200_COMM_BACKEND", "fused"),
    # ---- tuning switches of the kernel library and the communicator (docs/kernels.md,
    # docs/parallelism.md); each names the default in its second argument
    # programmatic dependent launch of the serving kernels (read once by the kernel library)
    "AB200_PDL": _flag("AB200_PDL", "0"),
    # split-K of one-row-of-tiles GEMMs inside thread-block clusters (0: through the workspace)
    "AB200_GEMM_CLUSTER": _flag("AB200_GEMM_CLUSTER", "1"),
    # fp8 codes stored in 16-row x 128-byte tiles instead of row-major
    "AB200_FP8_TILED": _flag("AB200_FP8_TILED", "0"),
    # small tensor-parallel reductions folded into the following RMSNorm kernel
    "AB200_FOLD_REDUCE": _flag("AB200_FOLD_REDUCE", "1"),
    # all-reduce kernel: "auto" (by size), "oneshot" or "twoshot"
    "AB200_ALLREDUCE": lambda: os.getenv("AB200_ALLREDUCE", "auto"),
    # a barrier kernel after every cross-rank exchange instead of signals and in-kernel waits
    "AB200_FUSED_BARRIERS": _flag("AB200_FUSED_BARRIERS", "0"),
    # long-lived engine objects frozen out of the cyclic garbage collector
    "AB200_GC_FREEZE": _flag("AB200_GC_FREEZE", "1"),
    # the speculator's n-head loop replayed from CUDA graphs
    "ARCTIC_B200_SPEC_GRAPH": _flag("ARCTIC_B200_SPEC_GRAPH", "1"),
}


def arctic_inference_effective_enabled(extra_env: Optional[dict] = None) -> bool:
    """True when the Arctic features are switched on for this process, either in its own
    environment or in the environment a launcher is about to hand to a worker."""
    if environment_variables["ARCTIC_INFERENCE_ENABLED"]():
        return True
    return bool(extra_env) and str(extra_env.get("ARCTIC_INFERENCE_ENABLED", "0")) == "1"


def __getattr__(name: str) -> Any:
    if name in environment_variables:
        return environment_variables[name]()
    raise AttributeError("Environment variable %r not found." % name)


def __dir__():
    return list(environment_variables)
