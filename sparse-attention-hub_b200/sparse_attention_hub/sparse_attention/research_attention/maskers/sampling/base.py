"""Sampling masker base (reference: .../maskers/sampling/base.py:13-48)."""

from abc import abstractmethod
from dataclasses import dataclass
from typing import Any, Dict

from ....utils.mask import Mask
from ..base import MaskerConfig, ResearchMasker


@dataclass
class SamplingMaskerConfig(MaskerConfig):
    """Base configuration for sampling maskers."""


class SamplingMasker(ResearchMasker):
    """Maskers whose entries carry sampling probabilities as weights."""

    def __init__(self, config: SamplingMaskerConfig) -> None:
        super().__init__(config)

    @abstractmethod
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        """Add sampling mask to attention computation."""

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "SamplingMasker":
        if not isinstance(config, SamplingMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
