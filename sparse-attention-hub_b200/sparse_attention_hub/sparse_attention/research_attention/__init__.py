"""Research attention: masker stacks over the native Mask."""

from .base import ResearchAttention, ResearchAttentionConfig

__all__ = ["ResearchAttention", "ResearchAttentionConfig"]
