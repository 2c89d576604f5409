"""Micro-metric logging."""

from .logger import LogEvent, MicroMetricLogger

__all__ = ["MicroMetricLogger", "LogEvent"]
