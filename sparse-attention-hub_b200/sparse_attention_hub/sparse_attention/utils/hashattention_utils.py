"""HashAttention weight files (reference: sparse_attention/utils/hashattention_utils.py:155-180).

A weight file is a pickle of `{layer_idx: {"query_matrix": [...], "query_bias": [...],
"key_matrix": [...], "key_bias": [...]}}` with one tensor per MLP layer, matrices
shaped `[heads, in, out]` and biases `[heads, out]`.
"""

import pickle
from typing import Dict, List

import torch

HatWeights = Dict[int, Dict[str, List[torch.Tensor]]]


def load_hat_weights(hat_weights_path: str, device: str = "cpu") -> HatWeights:
    """Load a HashAttention weight pickle and move every tensor to `device`."""
    with open(hat_weights_path, "rb") as f:
        weights: HatWeights = pickle.load(f)
    for layer_idx, layer in weights.items():
        for name, tensors in layer.items():
            weights[layer_idx][name] = [t.to(device) for t in tensors]
    return weights
