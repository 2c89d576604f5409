"""Maskers: registry, bases and the native implementations."""

from .base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry, ResearchMasker
from .fixed import *  # noqa: F401,F403  (registers the fixed maskers)
from .sampling import *  # noqa: F401,F403  (registers the sampling maskers)

__all__ = ["ResearchMasker", "MaskerConfig", "MaskerRegistry", "AttentionTensorDimensions"]
