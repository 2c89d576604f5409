"""Masker ABCs, config base and the config -> masker registry.

Reference: sparse_attention_hub/sparse_attention/research_attention/maskers/base.py
(:16-28 configs and dimensions, :31-85 registry, :88-208 ResearchMasker).
"""

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple, Type, TypeVar, Union

import torch

from ...utils.mask import Mask

T = TypeVar("T", bound="ResearchMasker")
ConfigType = TypeVar("ConfigType", bound="MaskerConfig")


@dataclass
class MaskerConfig:
    """Base configuration class for all maskers."""


@dataclass
class AttentionTensorDimensions:
    """Extents a masker needs: batch, query heads, query length, key length."""

    batch_size: int
    num_heads: int
    seq_len_queries: int
    seq_len_keys: int


class MaskerRegistry:
    """Maps a config dataclass to the masker class that consumes it."""

    _registry: Dict[Type[MaskerConfig], Type["ResearchMasker"]] = {}

    @classmethod
    def register(cls, config_type: Type[ConfigType]) -> Callable[[Type[T]], Type[T]]:
        """Class decorator: `@MaskerRegistry.register(MyConfig)`."""

        def decorator(masker_class: Type[T]) -> Type[T]:
            cls._registry[config_type] = masker_class
            return masker_class

        return decorator

    @classmethod
    def get_masker_class(cls, config_type: Type[MaskerConfig]) -> Type["ResearchMasker"]:
        masker_class = cls._registry.get(config_type)
        if masker_class is None:
            raise ValueError(f"No masker class registered for config type: {config_type}")
        return masker_class

    @classmethod
    def get_all_registered_types(cls) -> Dict[Type[MaskerConfig], Type["ResearchMasker"]]:
        return cls._registry.copy()


class ResearchMasker(ABC):
    """A step of the masker stack: extends `previous_mask` and returns the new `Mask`."""

    config: MaskerConfig

    def __init__(self, config: MaskerConfig) -> None:
        self.config = config

    def _extract_tensor_dimensions(self, keys: torch.Tensor,
                                   queries: torch.Tensor) -> AttentionTensorDimensions:
        return AttentionTensorDimensions(
            batch_size=queries.shape[0],
            num_heads=queries.shape[1],
            seq_len_queries=queries.shape[2],
            seq_len_keys=keys.shape[2],
        )

    @staticmethod
    def _mask_shape(dims: AttentionTensorDimensions) -> Tuple[int, int, int, int]:
        return (dims.batch_size, dims.num_heads, dims.seq_len_queries, dims.seq_len_keys)

    def _create_full_mask(self, dims: AttentionTensorDimensions, dtype: torch.dtype,
                          device: torch.device) -> Mask:
        return Mask.create_full_mask(self._mask_shape(dims), dtype=dtype, device=device)

    def _create_mask_from_rowise_indices(self, dims: AttentionTensorDimensions,
                                         indices: torch.Tensor, device: torch.device,
                                         dtype: torch.dtype) -> Mask:
        """Unit-weight mask from `[B, H, Sq, k]` column ids (dense scatter semantics)."""
        data = torch.ones_like(indices, dtype=dtype, device=device)
        return Mask.create_from_row_wise_idx(shape=self._mask_shape(dims), row_wise_idx=indices,
                                             data=data, mask_type="dense", dtype=dtype)

    def _refuse_sequence_shard(self, kwargs: Dict[str, Any]) -> None:
        """Maskers whose selection needs the whole sequence (a global top-k, a global sample
        budget) must not treat one rank's key range as all of it."""
        if kwargs.get("sequence_shard") is not None:
            raise NotImplementedError(
                f"{type(self).__name__} does not run on a sequence shard; "
                "Sink, Local, OracleTopK, HashAttention top-k and MagicPig do")

    def _calculate_effective_size(self, size_param: Union[float, int], seq_len_keys: int) -> int:
        """A float is a fraction of the key length (truncated), an int is a count."""
        if isinstance(size_param, float):
            return int(size_param * seq_len_keys)
        return int(size_param)

    @abstractmethod
    def add_mask(
        self,
        keys: torch.Tensor,
        queries: torch.Tensor,
        values: torch.Tensor,
        attention_mask: torch.Tensor,
        scaling: float,
        dropout: float,
        sparse_meta_data: Dict[Any, Any],
        previous_mask: Mask,
        **kwargs: Dict[str, Any],
    ) -> Mask:
        """Return `previous_mask` extended by this masker's selection."""

    @classmethod
    @abstractmethod
    def create_from_config(cls, config: MaskerConfig) -> "ResearchMasker":
        """Build the masker from its config dataclass."""

    @classmethod
    def create_masker_from_config(cls, config: MaskerConfig) -> "ResearchMasker":
        """Registry dispatch on `type(config)`; ValueError when nothing is registered."""
        masker_class: Optional[Type["ResearchMasker"]] = MaskerRegistry.get_masker_class(type(config))
        return masker_class.create_from_config(config)
