"""Native sampling maskers."""

from .adaptive_sampling import AdaptiveSamplingMasker, AdaptiveSamplingMaskerConfig
from .magic_pig import MagicPig, MagicPigConfig, PackedLSHSignatures
from .random_sampling import RandomSamplingMasker, RandomSamplingMaskerConfig

__all__ = ["AdaptiveSamplingMasker", "AdaptiveSamplingMaskerConfig", "MagicPig", "MagicPigConfig",
           "PackedLSHSignatures", "RandomSamplingMasker", "RandomSamplingMaskerConfig"]
