"""Sink, Local and Causal maskers on the device bitmap.

Reference: .../maskers/fixed/implementations/basic_fixed.py
(LocalMasker :37-277, CausalMasker :279-308, SinkMasker :329-462).

Both real maskers are a band fill on the bitmap (`sah_mask_fill_band`):
  Sink   columns [0, sink) of every row.
  Local  for query position q the columns j with
         S - Sq - W + 1 <= j - q < S - Sq + 1 are set, then the columns above
         the causal diagonal (j - q >= S - Sq + 1) are cleared, as the
         reference's default dense path does (basic_fixed.py:48-67).
A previous mask that carries non-unit weights takes the same edits on its
dense tensor instead.
"""

from dataclasses import dataclass, field
from typing import Any, Dict, Union

import torch

from ..... import _native_ops
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import FixedMasker, FixedMaskerConfig


@dataclass
class LocalMaskerConfig(FixedMaskerConfig):
    """`window_size`: count (int) or fraction of the key length (float), > 0."""

    window_size: Union[float, int]
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.window_size > 0:
            raise ValueError(f"window_size must be > 0, got {self.window_size}")


@MaskerRegistry.register(LocalMaskerConfig)
class LocalMasker(FixedMasker):
    """Keeps the `window_size` keys that end at each query's causal position."""

    window_size: Union[float, int]

    def __init__(self, config: LocalMaskerConfig) -> None:
        super().__init__(config)
        self.window_size = config.window_size

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        if previous_mask.is_full_mask():
            return previous_mask
        dims = self._extract_tensor_dimensions(keys, queries)
        # With a sequence shard the keys at hand are columns [begin, begin + S) of `total`
        # keys: sizes and the full-attention rule follow the whole sequence.
        shard = kwargs.get("sequence_shard")
        total = shard.total if shard is not None else dims.seq_len_keys
        window = self._calculate_effective_window_size(total)
        if total <= window + dims.seq_len_queries:
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        return self.get_updated_mask(dims, window, keys, previous_mask,
                                     key_offset=shard.begin if shard is not None else 0, total=total)

    def get_updated_mask(self, tensor_dims: AttentionTensorDimensions, effective_window_size: int,
                         keys: torch.Tensor, previous_mask: Mask, mode: str = "native",
                         key_offset: int = 0, total: int = None) -> Mask:
        S, Sq = tensor_dims.seq_len_keys, tensor_dims.seq_len_queries
        total = S if total is None else total
        band_lo = total - Sq - effective_window_size + 1 - key_offset
        band_hi = total - Sq + 1 - key_offset
        nb = _native_ops.unit_weight_bits(previous_mask)
        if nb is not None:
            _native_ops.fill_band(nb, Sq, band_lo, 1, band_hi, 1, 1)
            if Sq > 1:
                _native_ops.fill_band(nb, Sq, band_hi, 1, S, 0, 0)
            return Mask._from_native(previous_mask.shape, previous_mask.dtype,
                                     _native_ops.fresh_native(nb))
        dense = previous_mask.get_dense_mask()
        offset = (torch.arange(S, device=dense.device).unsqueeze(0)
                  - torch.arange(Sq, device=dense.device).unsqueeze(1))
        dense[..., (offset >= band_lo) & (offset < band_hi)] = 1.0
        dense[..., offset >= band_hi] = 0.0
        return Mask.create_mask_from_dense_mask(dense.shape, dense, previous_mask.dtype)

    def _calculate_effective_window_size(self, seq_len_keys: int) -> int:
        return self._calculate_effective_size(self.window_size, seq_len_keys)

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, window_size: int) -> bool:
        return dims.seq_len_keys <= window_size + dims.seq_len_queries

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "LocalMasker":
        if not isinstance(config, LocalMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)


@MaskerRegistry.register(FixedMaskerConfig)
class CausalMasker(FixedMasker):
    """Placeholder masker of the bare `FixedMaskerConfig`: returns the mask unchanged."""

    def __init__(self, config: FixedMaskerConfig) -> None:
        super().__init__(config)

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        return previous_mask

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "CausalMasker":
        if not isinstance(config, FixedMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)


@dataclass
class SinkMaskerConfig(FixedMaskerConfig):
    """`sink_size`: count (int) or fraction of the key length (float), > 0."""

    sink_size: Union[float, int]
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not self.sink_size > 0:
            raise ValueError(f"sink_size must be > 0, got {self.sink_size}")


@MaskerRegistry.register(SinkMaskerConfig)
class SinkMasker(FixedMasker):
    """Keeps the first `sink_size` keys of every row."""

    sink_size: Union[float, int]

    def __init__(self, config: SinkMaskerConfig) -> None:
        super().__init__(config)
        self.sink_size = config.sink_size

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        if previous_mask.is_full_mask():
            return previous_mask
        dims = self._extract_tensor_dimensions(keys, queries)
        shard = kwargs.get("sequence_shard")  # see LocalMasker.add_mask
        total = shard.total if shard is not None else dims.seq_len_keys
        sink = self._calculate_effective_sink_size(total)
        if total <= sink:
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        return self.get_updated_mask(dims, sink, keys, previous_mask,
                                     key_offset=shard.begin if shard is not None else 0)

    def get_updated_mask(self, tensor_dims: AttentionTensorDimensions, effective_sink_size: int,
                         keys: torch.Tensor, previous_mask: Mask, mode: str = "native",
                         key_offset: int = 0) -> Mask:
        nb = _native_ops.unit_weight_bits(previous_mask)
        hi = max(0, effective_sink_size - key_offset)
        if nb is not None:
            _native_ops.fill_band(nb, tensor_dims.seq_len_queries, 0, 0, hi, 0, 1)
            return Mask._from_native(previous_mask.shape, previous_mask.dtype,
                                     _native_ops.fresh_native(nb))
        dense = previous_mask.get_dense_mask()
        dense[..., :hi] = 1.0
        return Mask.create_mask_from_dense_mask(dense.shape, dense, previous_mask.dtype)

    def _calculate_effective_sink_size(self, seq_len_keys: int) -> int:
        return self._calculate_effective_size(self.sink_size, seq_len_keys)

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, sink_size: int) -> bool:
        return dims.seq_len_keys <= sink_size

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "SinkMasker":
        if not isinstance(config, SinkMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
