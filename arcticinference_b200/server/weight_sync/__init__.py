"""Weight synchronisation between a trainer (sender) and serving replicas (receivers)."""

from .schedule import TensorMeta, TransferSchedule  # noqa: F401
from .sender import WeightSender  # noqa: F401
