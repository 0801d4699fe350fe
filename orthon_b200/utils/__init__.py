"""Runtime utilities: GPU clock sampling and tracing ranges."""
from .clocks import ClockSampler  # noqa: F401
from .tracing import trace_range, enable_tracing, collected_ranges, timeline, clear_ranges, tracing_enabled  # noqa: F401
