"""Native sampling maskers."""

from .adaptive_sampling import AdaptiveSamplingMasker, AdaptiveSamplingMaskerConfig
from .random_sampling import RandomSamplingMasker, RandomSamplingMaskerConfig

__all__ = ["AdaptiveSamplingMasker", "AdaptiveSamplingMaskerConfig", "RandomSamplingMasker",
           "RandomSamplingMaskerConfig"]
