"""Oracle top-k: the k inactive keys with the largest unscaled q.k.

Reference: .../maskers/fixed/implementations/oracle_top_k.py (config :23-33,
update_core :48-80, add_mask :172-208).  Scores are q.k in the input dtype plus
the additive attention mask; positions already active in the previous mask do
not compete; winners get weight 1.  Two kernels: a K stream that scores every
key once for all query heads of its KV group, and an exact radix select with
ties to the lowest column.
"""

from dataclasses import dataclass, field
from typing import Any, Dict, Union

import torch

from ..... import _native_ops
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import TopKMasker, TopKMaskerConfig


@dataclass
class OracleTopKConfig(TopKMaskerConfig):
    """`heavy_size` keys per row; `search_space` is free-form tuning metadata."""

    search_space: Dict[str, Any] = field(default_factory=dict)


@MaskerRegistry.register(OracleTopKConfig)
class OracleTopK(TopKMasker):
    """Exact top-k of the true attention logits."""

    heavy_size: Union[float, int]

    def __init__(self, config: OracleTopKConfig) -> None:
        super().__init__(config)
        self.heavy_size = config.heavy_size

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        if previous_mask.is_full_mask():
            return previous_mask
        dims = self._extract_tensor_dimensions(keys, queries)
        # On a sequence shard the keys at hand are one rank's range: k and the full-attention
        # rule follow the whole sequence, and the top-k is global (exact, same tie rule).
        shard = kwargs.get("sequence_shard")
        total = shard.total if shard is not None else dims.seq_len_keys
        heavy = self._calculate_effective_heavy_size(total)
        if total <= heavy:
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        if shard is not None:
            if _native_ops.unit_weight_bits(previous_mask) is None:
                raise NotImplementedError("OracleTopK on a sequence shard needs a unit-weight previous mask")
            scores = self._compute_raw_attention_scores(keys, queries, attention_mask)
            merged = _native_ops.topk_select_sharded(scores, previous_mask, heavy, shard.comm)
            return Mask._from_native(previous_mask.shape, previous_mask.dtype, merged)
        return self.get_updated_mask(dims, heavy, keys, queries, attention_mask, previous_mask,
                                     call_cache=kwargs.get("_sah_call_cache"))

    def get_updated_mask(self, tensor_dims: AttentionTensorDimensions, effective_heavy_size: int,
                         keys: torch.Tensor, queries: torch.Tensor, attention_mask: torch.Tensor,
                         previous_mask: Mask, mode: str = "native", call_cache=None) -> Mask:
        scores = self._compute_raw_attention_scores(keys, queries, attention_mask)
        if call_cache is not None and attention_mask is None:
            # later maskers of the same call (adaptive sampling) need the same q.k stream
            call_cache["qk_scores"] = scores
        if _native_ops.unit_weight_bits(previous_mask) is None:
            # weighted previous mask: winners are written into its dense form
            merged = _native_ops.topk_select(scores, previous_mask, effective_heavy_size)
            new_only = _native_ops.bits_andnot(merged, previous_mask.native_bits())
            add = Mask._from_native(previous_mask.shape, previous_mask.dtype, new_only)
            dense = previous_mask.get_dense_mask()
            dense[add.get_dense_mask() != 0] = 1.0
            return Mask.create_mask_from_dense_mask(dense.shape, dense, previous_mask.dtype)
        merged = _native_ops.topk_select(scores, previous_mask, effective_heavy_size)
        return Mask._from_native(previous_mask.shape, previous_mask.dtype, merged)

    def _compute_raw_attention_scores(self, keys: torch.Tensor, queries: torch.Tensor,
                                      attention_mask: torch.Tensor,
                                      previous_dense_mask: torch.Tensor = None) -> torch.Tensor:
        """q.k (+ attention mask) in the input dtype, `[B, Hq, Sq, S]`."""
        return _native_ops.qk_scores(queries, keys, attention_mask)

    def _calculate_effective_heavy_size(self, seq_len_keys: int) -> int:
        return self._calculate_effective_size(self.heavy_size, seq_len_keys)

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, heavy_size: int) -> bool:
        return dims.seq_len_keys <= heavy_size

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "OracleTopK":
        if not isinstance(config, OracleTopKConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
