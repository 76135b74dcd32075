"""Shared utilities: measurement helpers (``measure``)."""
from .measure import ClockSampler, measured_peaks, time_cuda
