"""Sparse attention: base types, research attention, maskers, Mask."""

from .base import SparseAttention, SparseAttentionConfig
from .research_attention import ResearchAttention, ResearchAttentionConfig
from .research_attention.maskers import ResearchMasker
from .research_attention.maskers.fixed import (
    CausalMasker,
    FixedMasker,
    HashAttentionTopKMasker,
    HashAttentionTopKMaskerConfig,
    LocalMasker,
    LocalMaskerConfig,
    OracleTopK,
    OracleTopKConfig,
    OracleTopPMasker,
    OracleTopPMaskerConfig,
    PQCache,
    PQCacheConfig,
    QuestTopKMasker,
    QuestTopKMaskerConfig,
    SinkMasker,
    SinkMaskerConfig,
    TopKMasker,
    TopKMaskerConfig,
    TopPMasker,
)
from .research_attention.maskers.sampling import (
    AdaptiveSamplingMasker,
    AdaptiveSamplingMaskerConfig,
    MagicPig,
    MagicPigConfig,
    RandomSamplingMasker,
    RandomSamplingMaskerConfig,
    SamplingMasker,
)
from .utils import Mask

__all__ = [
    "SparseAttention", "SparseAttentionConfig", "ResearchAttention", "ResearchAttentionConfig",
    "ResearchMasker", "SamplingMasker", "FixedMasker", "TopKMasker", "TopKMaskerConfig",
    "TopPMasker", "LocalMasker", "LocalMaskerConfig", "CausalMasker", "SinkMasker",
    "SinkMaskerConfig", "OracleTopK", "OracleTopKConfig", "HashAttentionTopKMasker",
    "HashAttentionTopKMaskerConfig", "PQCache", "PQCacheConfig", "RandomSamplingMasker",
    "RandomSamplingMaskerConfig", "AdaptiveSamplingMasker", "AdaptiveSamplingMaskerConfig", "MagicPig",
    "MagicPigConfig", "OracleTopPMasker", "OracleTopPMaskerConfig", "QuestTopKMasker", "QuestTopKMaskerConfig", "Mask",
]
