"""Oracle top-p: the keys that carry the top `top_p` of a row's softmax mass.

Reference: .../maskers/fixed/implementations/oracle_top_p.py (config :23-33, add_mask
:47-78, full-attention rule :80-83, exp weights :85-106, thresholds :108-136, mask :138-169).
The weights are exp(scaling * q.k + attention_mask - row max) in the input dtype with the
previously active positions pushed to the lowest value; the threshold is the sorted weight at
which the normalised running sum passes `top_p`; every key whose weight reaches it is
selected.  One K stream for the logits (shared with OracleTopK) and one kernel per row set
that replaces the sort by a histogram over bfloat16 bit patterns.  bfloat16 inputs only.
"""

from dataclasses import dataclass, field
from typing import Any, Dict

import torch

from ..... import _native_ops
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import TopPMasker, TopPMaskerConfig


@dataclass
class OracleTopPMaskerConfig(TopPMaskerConfig):
    """`top_p`: the cumulative mass to cover; `search_space` is free-form tuning metadata."""

    search_space: Dict[str, Any] = field(default_factory=dict)


@MaskerRegistry.register(OracleTopPMaskerConfig)
class OracleTopPMasker(TopPMasker):
    """Exact top-p of the true attention weights."""

    def __init__(self, config: OracleTopPMaskerConfig) -> None:
        super().__init__(config)
        assert isinstance(self.top_p, float) and self.top_p is not None, \
            "top_p must be set as a float in config"

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        if previous_mask.is_full_mask():
            return previous_mask
        self._refuse_sequence_shard(kwargs)
        dims = self._extract_tensor_dimensions(keys, queries)
        if self._should_use_full_attention(dims):
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        return self._create_oracle_top_p_mask(dims, keys, queries, previous_mask, attention_mask,
                                              scaling, call_cache=kwargs.get("_sah_call_cache"))

    def _should_use_full_attention(self, dims: AttentionTensorDimensions) -> bool:
        return dims.seq_len_keys <= int(self.top_p * dims.seq_len_keys)

    def _create_oracle_top_p_mask(self, dims: AttentionTensorDimensions, keys: torch.Tensor,
                                  queries: torch.Tensor, previous_mask: Mask,
                                  attention_mask: torch.Tensor, scaling: float,
                                  call_cache=None) -> Mask:
        if queries.dtype != torch.bfloat16:
            raise NotImplementedError(
                "OracleTopPMasker runs in bfloat16 only: the reference accumulates a float32 row in "
                "float64 over values that do not fall into a small set")
        scores = None if call_cache is None else call_cache.get("qk_scores")
        if scores is None:
            scores = _native_ops.qk_scores(queries, keys, None)   # unscaled, no bias
            if call_cache is not None:
                call_cache["qk_scores"] = scores
        unit = _native_ops.unit_weight_bits(previous_mask) is not None
        sel = _native_ops.topp_select(scores, attention_mask, scaling, previous_mask, self.top_p,
                                      or_prev=unit)
        picked = Mask._from_native(previous_mask.shape, previous_mask.dtype, sel)
        if unit:
            return picked            # previous | selected, all weights 1
        return previous_mask.merge_mask(picked, inplace=False)

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "OracleTopPMasker":
        if not isinstance(config, OracleTopPMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
