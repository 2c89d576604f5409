"""Sampling maskers."""

from .base import SamplingMasker, SamplingMaskerConfig

__all__ = ["SamplingMasker", "SamplingMaskerConfig"]
