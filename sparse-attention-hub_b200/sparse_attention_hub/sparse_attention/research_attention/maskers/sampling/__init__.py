"""Sampling maskers."""

from .base import SamplingMasker, SamplingMaskerConfig
from .implementations import (
    AdaptiveSamplingMasker,
    AdaptiveSamplingMaskerConfig,
    MagicPig,
    MagicPigConfig,
    PackedLSHSignatures,
    RandomSamplingMasker,
    RandomSamplingMaskerConfig,
)

__all__ = ["SamplingMasker", "SamplingMaskerConfig", "RandomSamplingMasker",
           "RandomSamplingMaskerConfig", "AdaptiveSamplingMasker", "AdaptiveSamplingMaskerConfig",
           "MagicPig", "MagicPigConfig", "PackedLSHSignatures"]
