"""Logging, metric accumulation, experiment tracking and profiling (reference: lm_engine/logging_utils/*)."""

from .logger import log_environment, log_metrics, log_rank_0, print_rank_0, print_ranks_all, set_logger, warn_once, warn_rank_0
from .metrics import MetricsTrackingDict
from .profiler import StepProfiler
from .tracking import ExperimentsTracker
