"""Quest page top-k: the pages whose upper bound of q.k is largest, all of their keys selected.

Reference: .../maskers/fixed/implementations/quest_top_k.py (config :31-54, add_mask :72-106,
_create_quest_page_topk_mask :108-196, full-attention rule :198-202) and utils/quest_utils.py.
Per page and key channel the minimum and maximum over the page's keys; the page score is
sum_j max(q_j * min_j, q_j * max_j) in the input dtype; the best
`min(pages, max(3, heavy // page_size))` pages are expanded to their keys and joined with the
previous mask; under an additive attention mask, pages without an allowed key do not compete and
forbidden keys leave the mask.

The page bounds are an index over the keys like the hash codes of HashAttention: they live in
`sparse_meta_data["quest_pages"][layer_idx]`, per KV head, and only the pages touched by keys
appended since the previous call are recomputed (the reference recomputes all of them from the
keys at every call).  `label_bits` below 16 (pseudo-quantised bounds) is not implemented.
"""

from dataclasses import dataclass, field
from typing import Any, Dict

import torch

from ..... import _native_ops
from ....._native_ops import _native
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import TopKMasker, TopKMaskerConfig


@dataclass
class QuestTopKMaskerConfig(TopKMaskerConfig):
    """`heavy_size` keys per row in pages of `page_size`; `search_space` is free-form metadata."""

    page_size: int
    label_bits: int = 16
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        super().__post_init__()
        if not (0 < self.label_bits <= 16):
            raise ValueError(f"label_bits must be in range (0, 16], got {self.label_bits}")
        if self.page_size <= 0:
            raise ValueError("page_size must be greater than 0")


@MaskerRegistry.register(QuestTopKMaskerConfig)
class QuestTopKMasker(TopKMasker):
    """Quest page-top-k masker."""

    page_size: int
    label_bits: int

    def __init__(self, config: QuestTopKMaskerConfig) -> None:
        super().__init__(config)
        if config.page_size <= 0:
            raise ValueError("page_size must be a positive integer")
        self.page_size = int(config.page_size)
        self.heavy_size = config.heavy_size
        self.label_bits = config.label_bits

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        if previous_mask.is_full_mask():
            return previous_mask
        self._refuse_sequence_shard(kwargs)
        dims = self._extract_tensor_dimensions(keys, queries)
        heavy = self._calculate_effective_size(self.heavy_size, dims.seq_len_keys)
        if self._should_use_full_attention(dims, heavy):
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        if self.label_bits < 16:
            raise NotImplementedError("QuestTopKMasker: label_bits < 16 (pseudo-quantised page bounds) "
                                      "is not implemented")
        return self._create_quest_page_topk_mask(dims, heavy, keys, queries, attention_mask,
                                                 previous_mask, sparse_meta_data,
                                                 kwargs.get("layer_idx"))

    # ---- page bounds, kept between calls ---------------------------------------------------
    def _page_bounds(self, keys: torch.Tensor, sparse_meta_data, layer_idx):
        """(pmin, pmax, page capacity) for `keys`; pages touched by new keys are recomputed."""
        _native.require_cuda(keys, "keys")
        lib = _native.load()
        B, Hkv, S, D = keys.shape
        if D % 8 != 0:
            raise NotImplementedError(f"QuestTopKMasker: head dimension {D} (multiples of 8)")
        k = keys if keys.stride(-1) == 1 else keys.contiguous()
        ps = self.page_size
        P = -(-S // ps)
        state = None
        if sparse_meta_data is not None and layer_idx is not None:
            state = sparse_meta_data.setdefault("quest_pages", {}).get(layer_idx)
        usable = (state is not None and state["shape"] == (B, Hkv, D) and state["dtype"] == k.dtype
                  and state["page_size"] == ps and state["n_keys"] <= S and state["device"] == k.device)
        if not usable:
            cap = max(P + P // 2, 16)
            state = {"shape": (B, Hkv, D), "dtype": k.dtype, "page_size": ps, "n_keys": 0, "cap": cap,
                     "device": k.device,
                     # [B, Hkv, D/8, page capacity, 8]: eight channels of consecutive pages adjoin
                     "pmin": torch.empty((B, Hkv, D // 8, cap, 8), dtype=k.dtype, device=k.device),
                     "pmax": torch.empty((B, Hkv, D // 8, cap, 8), dtype=k.dtype, device=k.device)}
        elif P > state["cap"]:
            cap = P + P // 2
            for name in ("pmin", "pmax"):
                grown = torch.empty((B, Hkv, D // 8, cap, 8), dtype=k.dtype, device=k.device)
                grown[:, :, :, : state["cap"]] = state[name]
                state[name] = grown
            state["cap"] = cap
        first = state["n_keys"] // ps   # the page the first new key falls into
        if state["n_keys"] < S:
            _native.check(
                lib.sah_quest_page_minmax(k.data_ptr(), _native.dtype_code(k.dtype), k.stride(0), k.stride(1),
                                          k.stride(2), B, Hkv, S, D, ps, first, state["cap"],
                                          state["pmin"].data_ptr(), state["pmax"].data_ptr(),
                                          _native.stream_of(k.device)), "sah_quest_page_minmax")
            state["n_keys"] = S
        if sparse_meta_data is not None and layer_idx is not None:
            sparse_meta_data["quest_pages"][layer_idx] = state
        return state["pmin"], state["pmax"], state["cap"]

    def _create_quest_page_topk_mask(self, dims: AttentionTensorDimensions, heavy_tokens: int,
                                     keys: torch.Tensor, queries: torch.Tensor,
                                     attention_mask: torch.Tensor, previous_mask: Mask,
                                     sparse_meta_data=None, layer_idx=None) -> Mask:
        lib = _native.load()
        B, Hq, Sq, S = (dims.batch_size, dims.num_heads, dims.seq_len_queries, dims.seq_len_keys)
        D = queries.shape[-1]
        Hkv = keys.shape[1]
        ps = self.page_size
        P = -(-S // ps)
        pmin, pmax, cap = self._page_bounds(keys, sparse_meta_data, layer_idx)
        q = queries if queries.stride(-1) == 1 else queries.contiguous()
        dev = q.device
        st = _native.stream_of(dev)
        code = _native.dtype_code(q.dtype)
        keep, bptr, bsb, bsh, bsq = _native_ops.bias_args(attention_mask, q.dtype, S)
        scores = torch.empty((B, Hq, Sq, P), dtype=q.dtype, device=dev)
        _native.check(
            lib.sah_quest_scores(q.data_ptr(), code, q.stride(0), q.stride(1), q.stride(2), pmin.data_ptr(),
                                 pmax.data_ptr(), cap, B, Hq, Hkv, Sq, S, D, ps, bptr, bsb, bsh, bsq,
                                 scores.data_ptr(), st), "sah_quest_scores")
        k_pages = min(P, max(3, heavy_tokens // ps))
        if k_pages <= 0:
            k_pages = 1
        no_pages = Mask.create_empty_mask((B, Hq, Sq, P), previous_mask.dtype, dev)
        # bitmap over pages; rows of a few hundred to a few thousand page scores: one CTA each
        picked = _native_ops.topk_select(scores, no_pages, k_pages, per_row=(P <= 8192))
        unit = _native_ops.unit_weight_bits(previous_mask)
        prev = previous_mask.native_bits()
        out = _native_ops.NativeBits(torch.empty_like(prev.bits), prev.rows, S)
        if unit is None and attention_mask is not None:
            raise NotImplementedError("QuestTopKMasker: a weighted previous mask together with an "
                                      "attention mask is not implemented")
        _native.check(
            lib.sah_quest_expand(picked.bits.data_ptr(), picked.words,
                                 prev.bits.data_ptr() if unit is not None else None, bptr, code, bsb, bsh,
                                 bsq, B, Hq, Sq, S, prev.words, ps, out.bits.data_ptr(), st),
            "sah_quest_expand")
        del keep
        union = Mask._from_native(previous_mask.shape, previous_mask.dtype, out)
        if unit is not None:
            return union            # max(previous, pages), gated: all weights 1
        # weighted previous mask: max(previous, {0,1}) equals the clamped sum of a dense merge
        return previous_mask.merge_mask(union, inplace=False)

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, heavy_tokens: int) -> bool:
        return dims.seq_len_keys <= max(1, heavy_tokens)

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "QuestTopKMasker":
        if not isinstance(config, QuestTopKMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
