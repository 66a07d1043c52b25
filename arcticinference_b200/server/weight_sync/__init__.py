"""Weight synchronisation between a trainer (sender) and serving replicas (receivers)."""

from .schedule import SenderSchedule, TensorMeta, TransferGroup, TransferSchedule  # noqa: F401
from .sender import WeightSender  # noqa: F401

# the names of the reference's package (arctic_inference/server/weight_sync/__init__.py:34-48)
from .compat import (NCCLEngine, WeightInfo, build_weights_info, cleanup_shm,  # noqa: F401,E402
                     load_spec_checkpoint, load_weights_from_shm, save_weights_to_shm,
                     send_spec_weights, spec_bucket_size)

__all__ = ["NCCLEngine", "WeightSender", "TransferSchedule", "TransferGroup", "SenderSchedule",
           "TensorMeta", "WeightInfo",
           "build_weights_info", "load_spec_checkpoint", "spec_bucket_size", "send_spec_weights",
           "save_weights_to_shm", "load_weights_from_shm", "cleanup_shm"]
