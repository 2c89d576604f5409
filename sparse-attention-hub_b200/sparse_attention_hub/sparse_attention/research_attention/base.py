"""Research attention: a masker stack followed by masked attention.

Reference: sparse_attention_hub/sparse_attention/research_attention/base.py
(config :24-28, one-sampling-masker rule :52-59, custom_attention :63-170,
create_from_config :172-196).
"""

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
from torch import nn

from ...metric_logging.logger import MicroMetricLogger
from ..base import SparseAttention, SparseAttentionConfig
from ..utils.mask import Mask
from ..utils.mask_attention_utils import (
    get_masked_attention_output,
    get_true_attention_output,
)
from .maskers.base import MaskerConfig, ResearchMasker
from .maskers.sampling.base import SamplingMasker

MicroMetricLogger.register_metric("research_attention_density", float)
MicroMetricLogger.register_metric("research_attention_output_error", float)


@dataclass
class ResearchAttentionConfig(SparseAttentionConfig):
    """`masker_configs`: the stack, applied in order."""

    masker_configs: List[MaskerConfig]


class ResearchAttention(SparseAttention):
    """Runs every masker on the previous masker's `Mask`, then attends over the result."""

    maskers: List[ResearchMasker]

    #: The reference always materialises the dense `[B, Hq, Sq, Sk]` probability
    #: tensor as its second return value.  That is an O(Sk) write per row, which
    #: is what a sparse decode step avoids, so it is off unless asked for.
    return_attention_weights: bool = False

    def __init__(self, sparse_attention_config: SparseAttentionConfig,
                 maskers: List[ResearchMasker]) -> None:
        super().__init__(sparse_attention_config)
        if sum(1 for m in maskers if isinstance(m, SamplingMasker)) > 1:
            raise ValueError(
                "Only one sampling masker supported for efficiency; consider implementing all "
                "sampling logic in one masker"
            )
        self.maskers = maskers

    def build_mask(self, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                   attention_mask: Optional[torch.Tensor], scaling: float, dropout: float,
                   sparse_meta_data: Dict[Any, Any], **kwargs: Dict[str, Any]) -> Mask:
        """The masker loop alone: empty mask -> every masker in order."""
        shape = (queries.shape[0], queries.shape[1], queries.shape[2], keys.shape[2])
        mask = Mask.create_empty_mask(shape, dtype=queries.dtype, device=queries.device)
        # Scratch shared by the maskers of this one call (e.g. the q.k score stream that both
        # OracleTopK and adaptive sampling need); maskers that do not know the key ignore it.
        call_cache: Dict[str, Any] = {}
        for masker in self.maskers:
            mask = masker.add_mask(keys=keys, queries=queries, values=values,
                                   attention_mask=attention_mask, scaling=scaling,
                                   dropout=dropout, sparse_meta_data=sparse_meta_data,
                                   previous_mask=mask, _sah_call_cache=call_cache, **kwargs)
        return mask

    def custom_attention(self, module: Optional[nn.Module], queries: torch.Tensor,
                         keys: torch.Tensor, values: torch.Tensor,
                         attention_mask: Optional[torch.Tensor], scaling: float, dropout: float,
                         **kwargs: Dict[str, Any]) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if "sparse_meta_data" not in kwargs:
            raise ValueError(
                "sparse_meta_data must be provided in kwargs while calling custom_attention()"
            )
        sparse_meta_data: Dict[Any, Any] = kwargs.pop("sparse_meta_data")
        mask = self.build_mask(queries, keys, values, attention_mask, scaling, dropout,
                               sparse_meta_data, **kwargs)

        logger = MicroMetricLogger()
        if logger.is_metric_enabled("research_attention_density"):
            logger.log("research_attention_density", mask.get_density(),
                       metadata={"layer_idx": kwargs["layer_idx"]})

        s_aux_raw: Any = kwargs.pop("s_aux", None)
        s_aux = s_aux_raw if isinstance(s_aux_raw, torch.Tensor) else None
        result = get_masked_attention_output(
            module=module, queries=queries, keys=keys, values=values,
            attention_mask=attention_mask, sinks=s_aux, scaling=scaling, dropout=dropout,
            sparse_attention_mask=mask, return_attention_weights=self.return_attention_weights,
            **kwargs)
        if self.return_attention_weights:
            attention_output, attention_weights = result
        else:
            attention_output, attention_weights = result, None

        if logger.is_metric_enabled("research_attention_output_error"):
            true_out, _ = get_true_attention_output(module, queries, keys, values, attention_mask,
                                                    scaling, dropout, **kwargs)
            error = torch.norm(true_out - attention_output) / torch.norm(true_out)
            logger.log("research_attention_output_error", float(error.item()),
                       metadata={"layer_idx": kwargs["layer_idx"]})
        return attention_output, attention_weights

    @classmethod
    def create_from_config(cls, config: SparseAttentionConfig) -> "ResearchAttention":
        if not isinstance(config, ResearchAttentionConfig):
            raise TypeError(f"Expected ResearchAttentionConfig, got {type(config)}")
        maskers = [ResearchMasker.create_masker_from_config(c) for c in config.masker_configs]
        return cls(config, maskers)
