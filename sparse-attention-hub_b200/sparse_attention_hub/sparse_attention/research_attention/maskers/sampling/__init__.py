"""Sampling maskers."""

from .base import SamplingMasker, SamplingMaskerConfig
from .implementations import (
    AdaptiveSamplingMasker,
    AdaptiveSamplingMaskerConfig,
    RandomSamplingMasker,
    RandomSamplingMaskerConfig,
)

__all__ = ["SamplingMasker", "SamplingMaskerConfig", "RandomSamplingMasker",
           "RandomSamplingMaskerConfig", "AdaptiveSamplingMasker", "AdaptiveSamplingMaskerConfig"]
