"""GQA helpers (reference: sparse_attention_hub/sparse_attention/utils/kv_utils.py:5-45).

The native kernels never expand K/V: query head h reads KV head h // groups.
`repeat_kv` exists for user code that wants the expanded view.
"""

import torch


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """(batch, kv_heads, seq, dim) -> (batch, kv_heads * n_rep, seq, dim), each head repeated."""
    if n_rep == 1:
        return hidden_states
    return torch.repeat_interleave(hidden_states, repeats=n_rep, dim=1)


def _get_num_key_value_groups(queries: torch.Tensor, kv_tensor: torch.Tensor) -> int:
    """Query heads per KV head; ValueError when the head counts do not divide."""
    num_attention_heads: int = queries.shape[1]
    num_key_value_heads: int = kv_tensor.shape[1]
    if num_attention_heads % num_key_value_heads != 0:
        raise ValueError(
            f"num_attention_heads ({num_attention_heads}) must be divisible by "
            f"num_key_value_heads ({num_key_value_heads})"
        )
    return num_attention_heads // num_key_value_heads
