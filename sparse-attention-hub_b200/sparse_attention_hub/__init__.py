"""B200-native decode-time research attention behind the sparse-attention-hub API.

The import paths, class names and call signatures of the hot path follow
skylight-org/sparse-attention-hub (`sparse_attention_hub.sparse_attention...`);
the work runs in hand-written sm_100a CUDA kernels reached through the C ABI of
`libsah_b200.so` (see `_native.py`).
"""

__version__ = "0.1.0"

from .metric_logging import MicroMetricLogger
from .sparse_attention import ResearchAttention, SparseAttention

__all__ = ["SparseAttention", "ResearchAttention", "MicroMetricLogger"]
