"""Native fixed maskers."""

from .basic_fixed import (
    CausalMasker,
    LocalMasker,
    LocalMaskerConfig,
    SinkMasker,
    SinkMaskerConfig,
)
from .hashattention_top_k import HashAttentionTopKMasker, HashAttentionTopKMaskerConfig
from .oracle_top_k import OracleTopK, OracleTopKConfig
from .oracle_top_p import OracleTopPMasker, OracleTopPMaskerConfig
from .pq_top_k import PQCache, PQCacheConfig
from .quest_top_k import QuestTopKMasker, QuestTopKMaskerConfig

__all__ = [
    "LocalMasker", "CausalMasker", "SinkMasker", "OracleTopK", "HashAttentionTopKMasker",
    "LocalMaskerConfig", "SinkMaskerConfig", "OracleTopKConfig", "HashAttentionTopKMaskerConfig",
    "PQCache", "PQCacheConfig", "OracleTopPMasker", "OracleTopPMaskerConfig", "QuestTopKMasker", "QuestTopKMaskerConfig",
]
