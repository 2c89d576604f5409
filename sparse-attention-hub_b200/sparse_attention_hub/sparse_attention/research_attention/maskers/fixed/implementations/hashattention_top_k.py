"""HashAttention top-k on packed sign-bit signatures.

Reference: .../maskers/fixed/implementations/hashattention_top_k.py (config
:26-42, add_mask :79-127, signatures :203-253, key cache :255-341, score
:343-371).  A signature is sign(MLP(x)) with one MLP per query head; keys are
hashed with the weights of every query head of their KV group.  The reference
keeps signatures as +-1 tensors and scores with a matmul; here a signature is
one uint32 per (batch, query head, key), the score is
bits - 2 * popcount(q ^ k), and the exact top-k (ties to the lowest column) is
a counting select over at most bits + 1 distinct scores.

`sparse_meta_data["key"][layer_idx]` holds a `PackedKeySignatures`; it grows
when the key length grows and only the new keys are hashed (:294-341).
"""

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union

import torch

from ..... import _native_ops
from .....utils.hashattention_utils import load_hat_weights
from .....utils.kv_utils import _get_num_key_value_groups
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import TopKMasker, TopKMaskerConfig


@dataclass
class HashAttentionTopKMaskerConfig(TopKMaskerConfig):
    """HashAttention parameters; exactly one of `hat_weights` / `hat_weight_file`."""

    hat_bits: int
    hat_mlp_layers: int
    hat_mlp_hidden_size: int
    hat_mlp_activation: str
    hat_weights: Optional[Dict[int, Dict[str, List[torch.Tensor]]]] = None
    hat_weight_file: Optional[str] = None
    search_space: Dict[str, Any] = field(default_factory=dict)


class PackedKeySignatures:
    """Packed key signatures of one layer: int32 words `[B, Hq, capacity]`, `length` valid."""

    def __init__(self, codes: torch.Tensor, length: int) -> None:
        self.codes = codes
        self.length = length

    @property
    def shape(self) -> Tuple[int, ...]:
        return (self.codes.shape[0], self.codes.shape[1], self.length)


@MaskerRegistry.register(HashAttentionTopKMaskerConfig)
class HashAttentionTopKMasker(TopKMasker):
    """Top-k by Hamming similarity of learned hash signatures."""

    heavy_size: Union[float, int]
    hat_bits: int
    hat_mlp_layers: int
    hat_mlp_hidden_size: int
    hat_mlp_activation: str
    hat_weights: Dict[int, Dict[str, List[torch.Tensor]]]

    def __init__(self, config: HashAttentionTopKMaskerConfig) -> None:
        super().__init__(config)
        self.heavy_size = config.heavy_size
        self.hat_bits = config.hat_bits
        self.hat_mlp_layers = config.hat_mlp_layers
        self.hat_mlp_hidden_size = config.hat_mlp_hidden_size
        self.hat_mlp_activation = config.hat_mlp_activation
        if config.hat_weights is not None and config.hat_weight_file is not None:
            raise ValueError("Only one of hat_weights or hat_weight_file should be provided")
        if config.hat_weights is None and config.hat_weight_file is None:
            raise ValueError("Either hat_weights or hat_weight_file must be provided")
        if config.hat_weight_file is not None:
            self.hat_weights = load_hat_weights(config.hat_weight_file)
        else:
            self.hat_weights = config.hat_weights
        self._prepared: Dict[Tuple, Tuple[List[torch.Tensor], List[torch.Tensor]]] = {}

    # ------------------------------------------------------------------ public
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[str, Dict[int, Any]], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        layer_idx = self._validate_inputs(sparse_meta_data, kwargs)
        if previous_mask.is_full_mask():
            return previous_mask
        dims = self._extract_tensor_dimensions(keys, queries)
        # On a sequence shard the keys at hand are one rank's range: k and the full-attention
        # rule follow the whole sequence, and the top-k is global (exact, same tie rule).
        shard = kwargs.get("sequence_shard")
        total = shard.total if shard is not None else dims.seq_len_keys
        heavy = self._calculate_effective_heavy_size(total)
        if total <= heavy:
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        if self.hat_mlp_activation not in ("relu", "silu", "gelu", "tanh"):
            raise ValueError(f"Unsupported activation function: {self.hat_mlp_activation}")
        _get_num_key_value_groups(queries, keys)

        key_sig = self._update_key_signatures(keys, queries.shape[1], sparse_meta_data, layer_idx)
        query_codes = self._encode(queries, queries.shape[1], layer_idx, "query")
        shape = self._mask_shape(dims)
        if shard is not None:
            if attention_mask is not None:
                raise NotImplementedError(
                    "HashAttention top-k on a sequence shard takes no additive attention mask")
            merged = _native_ops.hash_topk_sharded(key_sig.codes, query_codes, self.hat_bits,
                                                   previous_mask, heavy, shape, shard.comm)
        else:
            merged = _native_ops.hash_topk(key_sig.codes, key_sig.length, query_codes, self.hat_bits,
                                           attention_mask, queries.dtype, previous_mask, heavy, shape)
        if _native_ops.unit_weight_bits(previous_mask) is None:
            new_only = _native_ops.bits_andnot(merged, previous_mask.native_bits())
            add = Mask._from_native(shape, previous_mask.dtype, new_only)
            return previous_mask.merge_mask(add, inplace=False)
        return Mask._from_native(shape, previous_mask.dtype, merged)

    # --------------------------------------------------------------- internals
    def _validate_inputs(self, sparse_meta_data, kwargs: Dict[str, Any]) -> int:
        if sparse_meta_data is None:
            raise ValueError("sparse_meta_data cannot be None")
        layer_idx = kwargs.get("layer_idx")
        if layer_idx is None:
            raise ValueError("layer_idx must be provided in kwargs")
        return layer_idx

    def _layer_weights(self, layer_idx: int, tensor_type: str, device: torch.device,
                       dtype: torch.dtype) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
        """Contiguous `[H, in, out]` matrices and `[H, out]` biases on `device` in `dtype`."""
        key = (layer_idx, tensor_type, str(device), dtype)
        if key not in self._prepared:
            layer = self.hat_weights[layer_idx]
            mats = [m.to(device=device, dtype=dtype).contiguous() for m in layer[f"{tensor_type}_matrix"]]
            bias = [b.to(device=device, dtype=dtype).contiguous() for b in layer[f"{tensor_type}_bias"]]
            self._prepared[key] = (mats, bias)
        return self._prepared[key]

    def _encode(self, x: torch.Tensor, n_heads_out: int, layer_idx: int, tensor_type: str,
                codes: Optional[torch.Tensor] = None, n_begin: int = 0,
                n_end: Optional[int] = None) -> torch.Tensor:
        mats, bias = self._layer_weights(layer_idx, tensor_type, x.device, x.dtype)
        n_end = x.shape[2] if n_end is None else n_end
        if codes is None:
            codes = torch.empty((x.shape[0], n_heads_out, x.shape[2]), dtype=torch.int32,
                                device=x.device)
        _native_ops.hash_encode(x, n_heads_out, mats, bias, self.hat_mlp_activation, codes,
                                n_begin, n_end)
        return codes

    def _update_key_signatures(self, keys: torch.Tensor, n_query_heads: int,
                               sparse_meta_data: Dict[str, Dict[int, Any]],
                               layer_idx: int) -> PackedKeySignatures:
        cache = sparse_meta_data.setdefault("key", {})
        cached: Optional[PackedKeySignatures] = cache.get(layer_idx)
        n_keys = keys.shape[2]
        if cached is not None and not isinstance(cached, PackedKeySignatures):
            raise TypeError(
                "sparse_meta_data['key'] holds a foreign object; this masker stores "
                "PackedKeySignatures there")
        if cached is None:
            codes = torch.empty((keys.shape[0], n_query_heads, _capacity_for(n_keys)),
                                dtype=torch.int32, device=keys.device)
            cached = PackedKeySignatures(codes, 0)
        if n_keys < cached.length:
            raise ValueError(
                f"Current number of keys ({n_keys}) is less than cached number of keys "
                f"({cached.length})")
        if n_keys > cached.length:
            if n_keys > cached.codes.shape[-1]:
                grown = torch.empty((keys.shape[0], n_query_heads, _capacity_for(n_keys)),
                                    dtype=torch.int32, device=keys.device)
                grown[..., : cached.length] = cached.codes[..., : cached.length]
                cached.codes = grown
            self._encode(keys, n_query_heads, layer_idx, "key", cached.codes, cached.length, n_keys)
            cached.length = n_keys
        cache[layer_idx] = cached
        return cached

    def _calculate_effective_heavy_size(self, seq_len_keys: int) -> int:
        return self._calculate_effective_size(self.heavy_size, seq_len_keys)

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, heavy_size: int) -> bool:
        return dims.seq_len_keys <= heavy_size

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "HashAttentionTopKMasker":
        if not isinstance(config, HashAttentionTopKMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)


def _capacity_for(n_keys: int) -> int:
    """Room for decode-time appends without reallocating every step."""
    return n_keys + max(256, n_keys // 16)
