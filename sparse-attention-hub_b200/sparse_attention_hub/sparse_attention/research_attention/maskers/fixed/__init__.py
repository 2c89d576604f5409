"""Fixed-pattern maskers."""

from .base import (
    FixedMasker,
    FixedMaskerConfig,
    TopKMasker,
    TopKMaskerConfig,
    TopPMasker,
    TopPMaskerConfig,
)
from .implementations import (
    CausalMasker,
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
)

__all__ = [
    "FixedMasker", "TopKMasker", "TopPMasker", "FixedMaskerConfig", "TopKMaskerConfig",
    "TopPMaskerConfig", "LocalMasker", "CausalMasker", "SinkMasker", "OracleTopK",
    "HashAttentionTopKMasker", "LocalMaskerConfig", "SinkMaskerConfig", "OracleTopKConfig",
    "HashAttentionTopKMaskerConfig", "PQCache", "PQCacheConfig", "OracleTopPMasker", "OracleTopPMaskerConfig", "QuestTopKMasker", "QuestTopKMaskerConfig",
]
