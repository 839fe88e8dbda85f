"""Debug and observability helpers (opt-in; none of them is imported on the hot path)."""
from .hooks import GraphInputWatcher, LoggingOps, ModuleTracer, StageTimer  # noqa: F401
from .logging import init_logger, redirect_rank_output  # noqa: F401
from .profiling import nvtx_range, profiler_window  # noqa: F401
