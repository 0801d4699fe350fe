"""Runtime utilities: GPU clock sampling, timers, NVTX-style tracing ranges."""
from .clocks import ClockSampler  # noqa: F401
from .tracing import trace_range, enable_tracing, collected_ranges  # noqa: F401
