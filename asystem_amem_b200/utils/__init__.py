"""Timing, clock sampling and roofline helpers shared by the benches."""
from .timing import ClockSampler, cuda_time_ms, load_measured_peaks, max_over_ranks  # noqa: F401
