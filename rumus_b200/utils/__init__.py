from .metrics import MetricsLogger, DeviceTimer, trace_range
from .config import (PRESETS, ModelPreset, ParallelConfig, PrecisionConfig, TrainConfig, load_config)
from .fault import (Heartbeat, PeerLost, FaultInjector, check_device_status)
from .elastic import ElasticSupervisor, latest_checkpoint
from .canary import CanaryError, canary_guard  # noqa: E402,F401
