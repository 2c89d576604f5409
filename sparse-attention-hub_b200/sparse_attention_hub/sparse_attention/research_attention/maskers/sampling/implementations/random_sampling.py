"""Uniform random sampling of key positions with the sampling rate as weight.

Reference: .../maskers/sampling/implementations/random_sampling.py (config :27-48,
add_mask :95-193): `int(rate * S)` columns per row drawn with replacement from
[0, S), each carrying weight `rate`; merged into the previous mask with
clamp(previous + sampled, 0, 1), so duplicates collapse and positions that were
already active keep weight 1.

The draws come from `torch.randint` on the keys' device, or -- so that two
implementations can be fed the same sample -- from
`sparse_meta_data["random_sampling_draws"][layer_idx]` (int64 `[B, H, Sq, n]`).
"""

from dataclasses import dataclass, field
from typing import Any, Dict

import torch

from ..... import _native_ops
from .....utils.mask import Mask
from ...base import MaskerConfig, MaskerRegistry
from ..base import SamplingMasker, SamplingMaskerConfig


@dataclass
class RandomSamplingMaskerConfig(SamplingMaskerConfig):
    """`sampling_rate` in (0, 1]: fraction of the keys to draw per row."""

    sampling_rate: float
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not (0.0 < self.sampling_rate <= 1.0):
            raise ValueError(f"sampling_rate must be in range (0, 1], got {self.sampling_rate}")


@MaskerRegistry.register(RandomSamplingMaskerConfig)
class RandomSamplingMasker(SamplingMasker):
    """Adds `int(rate * S)` uniformly drawn keys per row, weighted by `rate`."""

    sampling_rate: float

    def __init__(self, config: RandomSamplingMaskerConfig) -> None:
        super().__init__(config)
        self.sampling_rate = config.sampling_rate

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        self._refuse_sequence_shard(kwargs)
        if previous_mask.is_full_mask():
            return previous_mask
        B, H, Sq = queries.shape[0], queries.shape[1], queries.shape[2]
        S = keys.shape[2]
        n = int(self.sampling_rate * S)
        if n <= 0:
            raise ValueError("row_wise_idx must have at least one column")
        rows = B * H * Sq
        layer_idx = kwargs.get("layer_idx")
        draws = None
        if sparse_meta_data is not None:
            draws = sparse_meta_data.get("random_sampling_draws", {}).get(layer_idx)
        if draws is None:
            draws = torch.randint(low=0, high=S, size=(B, H, Sq, n), device=keys.device,
                                  dtype=torch.long)
        cols = draws.to(device=keys.device, dtype=torch.long).reshape(rows * n)
        sptr = torch.arange(0, rows * n + 1, n, dtype=torch.long, device=keys.device)
        weight = torch.full((rows,), self.sampling_rate, dtype=previous_mask.dtype, device=keys.device)
        return _native_ops.merge_sampled(previous_mask, cols, sptr, weight)

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "RandomSamplingMasker":
        if not isinstance(config, RandomSamplingMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
