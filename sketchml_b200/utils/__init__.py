"""Timers, metrics, checkpoints, model export and roofline arithmetic."""
from .timing import PhaseTimer, cuda_time_ms  # noqa: F401
from .metrics import MetricsLogger, get_logger, rank_sum_auc  # noqa: F401
from .checkpoint import save_checkpoint, load_checkpoint, export_model, import_model, weights_hash  # noqa: F401
from .roofline import load_peaks, roofline_fraction  # noqa: F401
