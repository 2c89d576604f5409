"""Fixed-pattern and top-k masker bases.

Reference: .../maskers/fixed/base.py (:13-48 FixedMasker, :51-107 TopKMasker,
:110-152 TopPMasker).  `TopKMasker._native_topk` is the shared device path:
scores -> exact top-k over the positions the previous mask leaves inactive,
ties to the lowest column, winners OR-ed into the previous bitmap.
"""

from abc import abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, Union

import torch

from .... import _native_ops
from ....utils.mask import Mask
from ..base import MaskerConfig, ResearchMasker


@dataclass
class FixedMaskerConfig(MaskerConfig):
    """Base configuration for fixed pattern maskers."""


class FixedMasker(ResearchMasker):
    """Maskers whose selection does not involve randomness."""

    def __init__(self, config: FixedMaskerConfig) -> None:
        super().__init__(config)

    @abstractmethod
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        """Add fixed mask to attention computation."""

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "FixedMasker":
        if not isinstance(config, FixedMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)


@dataclass
class TopKMaskerConfig(FixedMaskerConfig):
    """`heavy_size`: count (int) or fraction of the key length (float)."""

    heavy_size: Union[float, int]

    def __post_init__(self) -> None:
        if not self.heavy_size > 0:
            raise ValueError(f"heavy_size must be > 0, got {self.heavy_size}")


class TopKMasker(FixedMasker):
    """Maskers that add the k best-scoring inactive positions of every row."""

    def __init__(self, config: TopKMaskerConfig) -> None:
        super().__init__(config)

    def _get_topk_indices_from_inactive_positions(self, scores: torch.Tensor, previous_mask: Mask,
                                                  k: int) -> torch.Tensor:
        """`[B, H, Sq, k]` ascending column ids of the top-k inactive positions.

        Same contract as the reference helper (fixed/base.py:74-85) with the tie
        rule made explicit: among equal scores the lowest column wins.
        """
        shape = tuple(scores.shape)
        merged = _native_ops.topk_select(scores, previous_mask, k)
        prev = previous_mask.native_bits()
        new_only = Mask._from_native(shape, previous_mask.dtype,
                                     _native_ops.bits_andnot(merged, prev))
        idx, ptr, _ = new_only.get_index_mask()
        cols = idx % shape[-1]
        return cols.reshape(shape[:-1] + (-1,))

    @abstractmethod
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        """Add top-K mask to attention computation."""

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "TopKMasker":
        if not isinstance(config, TopKMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)


@dataclass
class TopPMaskerConfig(FixedMaskerConfig):
    """`top_p` in [0, 1]."""

    top_p: float

    def __post_init__(self) -> None:
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError(f"top_p must be in range [0, 1], got {self.top_p}")


class TopPMasker(FixedMasker):
    """Abstract base of cumulative-mass maskers."""

    def __init__(self, config: TopPMaskerConfig) -> None:
        super().__init__(config)
        self.top_p: float = config.top_p

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "TopPMasker":
        if not isinstance(config, TopPMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
