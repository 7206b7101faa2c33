"""Checkpointing, logging / metrics, timeline tracing and host-side failure detection."""
from .ckpt import load_checkpoint, save_checkpoint  # noqa: F401
from .health import HealthMonitor, PeerFailure  # noqa: F401
from .logging import MetricsWriter, engine_metrics, setup_logging  # noqa: F401
from .timeline import Timeline, nvtx_range  # noqa: F401
