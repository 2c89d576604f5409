"""Sparse-attention base types (reference: sparse_attention_hub/sparse_attention/base.py:10-75)."""

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn


@dataclass
class SparseAttentionConfig:
    """Base configuration of a sparse attention mechanism."""


class SparseAttention(ABC):
    """Interface the HuggingFace hook calls: `custom_attention(...) -> (output, weights)`."""

    sparse_attention_config: SparseAttentionConfig

    def __init__(self, sparse_attention_config: SparseAttentionConfig) -> None:
        self.sparse_attention_config = sparse_attention_config

    @abstractmethod
    def custom_attention(
        self,
        module: nn.Module,
        queries: torch.Tensor,
        keys: torch.Tensor,
        values: torch.Tensor,
        attention_mask: Optional[torch.Tensor],
        scaling: float,
        dropout: float,
        **kwargs: Dict[str, Any],
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Attention output `[B, Sq, Hq, D]` and optional attention weights."""

    def pre_attention_hook_generator(self) -> None:
        """Kept for interface parity; nothing to install."""

    @classmethod
    def create_from_config(cls, config: SparseAttentionConfig) -> "SparseAttention":
        """Route a config to the mechanism that handles it."""
        from .research_attention import ResearchAttention, ResearchAttentionConfig

        if isinstance(config, ResearchAttentionConfig):
            return ResearchAttention.create_from_config(config)
        return cls(config)
