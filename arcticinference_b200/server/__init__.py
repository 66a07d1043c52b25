"""Replica-pool serving: REST API, request scheduler, workers, metrics, weight sync."""


def ensure_ray(*args, **kwargs) -> None:
    """Replicas are child processes here, not Ray actors: there is nothing to start. Kept so
    that launch scripts written for the reference (arctic_inference/server/__init__.py) run."""
    return None


def __getattr__(name: str):
    # resolved on first use: importing the package must not pull in FastAPI or torch.distributed
    if name == "ModelConfig":
        from .config import ModelConfig
        return ModelConfig
    if name == "Pipeline":
        from .pipeline import Pipeline
        return Pipeline
    if name == "ReplicaPool":
        from .replica_pool import ReplicaPool
        return ReplicaPool
    if name in ("NCCLEngine", "WeightInfo", "build_weights_info"):
        from . import weight_sync
        return getattr(weight_sync, name)
    raise AttributeError(name)


__all__ = ["ModelConfig", "Pipeline", "ReplicaPool", "ensure_ray", "NCCLEngine", "WeightInfo",
           "build_weights_info"]
