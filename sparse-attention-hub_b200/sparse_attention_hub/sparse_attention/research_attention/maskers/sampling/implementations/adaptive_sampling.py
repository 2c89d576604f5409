"""Adaptive (epsilon, delta) sampling (vAttention).

Reference: .../maskers/sampling/implementations/adaptive_sampling.py (config
:35-120, range :203-228, base count :230-235, std estimate :237-280, budget
:282-302, add_mask :304-407) and utils/mask_attention_utils.py:105-184.

Per row: a base sample of the exp-attention weights in [init_offset, S -
local_offset) estimates their spread and the softmax denominator; the budget
that bounds the denominator error by epsilon with confidence 1 - delta is
(ppf(1 - delta) * std * n / (epsilon * denominator))^2, clamped to [base count,
n]; that many columns are drawn uniformly with replacement and carry weight
budget / n.  The base sample is only used for the estimate.

One kernel per row computes the budget from the q.k scores (shared with an
OracleTopK masker earlier in the stack when there is no attention mask), a second
scatters the draws into a bitmap, and the sampled set is merged with
clamp(previous + p, 0, 1).  Draws are Philox4x32-10 of (seed, index):
`sparse_meta_data["adaptive_sampling_seed"]` (default 0) mixed with the layer and
a per-layer call counter; explicit draws can be handed in through
`sparse_meta_data["adaptive_sampling_draws"][layer] = {"base": [B,H,Sq,nb], "pool": [N]}`.
"""

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple, Union

import torch
from scipy.stats import norm

from ..... import _native_ops
from ....._native_ops import _native
from .....utils.mask import Mask, words_per_row
from ...base import MaskerConfig, MaskerRegistry
from ..base import SamplingMasker, SamplingMaskerConfig


@dataclass
class AdaptiveSamplingMaskerConfig(SamplingMaskerConfig):
    """base_rate_sampling: float in [0,1) or int >= 0; epsilon, delta in (0,1);
    init_offset / local_offset: int >= 0 or float fraction of the key length in [0,1]."""

    base_rate_sampling: Union[int, float]
    epsilon: float
    delta: float
    init_offset: Union[int, float]
    local_offset: Union[int, float]
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if isinstance(self.base_rate_sampling, float):
            if not (0.0 <= self.base_rate_sampling < 1.0):
                raise ValueError(
                    f"base_rate_sampling must be in [0, 1) if float, got {self.base_rate_sampling}")
        elif isinstance(self.base_rate_sampling, int):
            if self.base_rate_sampling < 0:
                raise ValueError(
                    f"base_rate_sampling must be non-negative if int, got {self.base_rate_sampling}")
        else:
            raise ValueError(
                f"base_rate_sampling must be int or float, got {type(self.base_rate_sampling)}")
        if not (0.0 < self.epsilon < 1.0):
            raise ValueError(f"epsilon must be in (0, 1), got {self.epsilon}")
        if not (0.0 < self.delta < 1.0):
            raise ValueError(f"delta must be in (0, 1), got {self.delta}")
        for name in ("init_offset", "local_offset"):
            val = getattr(self, name)
            if isinstance(val, float):
                if not (0.0 <= val <= 1.0):
                    raise ValueError(f"{name} must be in [0, 1] if float, got {val}")
            elif isinstance(val, int):
                if val < 0:
                    raise ValueError(f"{name} must be non-negative if int, got {val}")
            else:
                raise ValueError(f"{name} must be int or float, got {type(val)}")


@MaskerRegistry.register(AdaptiveSamplingMaskerConfig)
class AdaptiveSamplingMasker(SamplingMasker):
    """Budgeted uniform sampling with statistical error control."""

    def __init__(self, config: AdaptiveSamplingMaskerConfig) -> None:
        super().__init__(config)
        self.base_rate_sampling = config.base_rate_sampling
        self.epsilon = config.epsilon
        self.delta = config.delta
        self.init_offset = config.init_offset
        self.local_offset = config.local_offset
        self.delta_ppf = float(norm.ppf(1 - self.delta))

    def should_return_full_mask(self, sampling_range: int) -> bool:
        return sampling_range < 2

    def _get_sampling_range(self, seq_len_keys: int) -> Tuple[int, int, int]:
        start = int(self.init_offset * seq_len_keys) if isinstance(self.init_offset, float) \
            else self.init_offset
        end = seq_len_keys - (int(self.local_offset * seq_len_keys)
                              if isinstance(self.local_offset, float) else self.local_offset)
        return start, end, end - start

    def _get_base_sample_count(self, sampling_range: int) -> int:
        if isinstance(self.base_rate_sampling, int):
            return max(2, self.base_rate_sampling)
        return max(2, int(self.base_rate_sampling * sampling_range))

    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        self._refuse_sequence_shard(kwargs)
        if previous_mask.is_full_mask():
            return previous_mask
        if self.base_rate_sampling == 0:
            return previous_mask
        B, H, Sq = queries.shape[0], queries.shape[1], queries.shape[2]
        S = keys.shape[2]
        start, end, n = self._get_sampling_range(S)
        if self.should_return_full_mask(n):
            return Mask.create_full_mask((B, H, Sq, S), previous_mask.dtype, previous_mask.device)
        _native.require_cuda(keys, "keys")
        lib = _native.load()
        dev = keys.device
        st = _native.stream_of(dev)
        dtype = queries.dtype
        rows = B * H * Sq
        nb = self._get_base_sample_count(n)
        layer_idx = kwargs.get("layer_idx", 0)

        # unscaled, unbiased q.k: the same tensor an OracleTopK earlier in the stack computed
        cache: Optional[dict] = kwargs.get("_sah_call_cache")
        scores = cache.get("qk_scores") if cache is not None else None
        if scores is None:
            scores = _native_ops.qk_scores(queries, keys, None)
            if cache is not None:
                cache["qk_scores"] = scores

        meta = sparse_meta_data if sparse_meta_data is not None else {}
        seed = int(meta.get("adaptive_sampling_seed", 0))
        calls = meta.setdefault("adaptive_sampling_calls", {})
        call_no = calls.get(layer_idx, 0)
        calls[layer_idx] = call_no + 1
        base_seed = (seed * 1000003 + layer_idx * 7919 + call_no * 2) & 0xFFFFFFFFFFFFFFFF
        handed = meta.get("adaptive_sampling_draws", {}).get(layer_idx) or {}
        base_draws = handed.get("base")
        pool = handed.get("pool")
        if base_draws is not None:
            base_draws = base_draws.to(device=dev, dtype=torch.long).reshape(rows, nb).contiguous()
        if pool is not None:
            pool = pool.to(device=dev, dtype=torch.long).contiguous()

        if previous_mask.is_empty:
            prev_nb = None
        else:
            prev_nb = previous_mask.native_bits()
            if prev_nb.data is not None:
                prev_nb.ensure_scan()
        keep, bptr, bsb, bsh, bsq = _native_ops.bias_args(attention_mask, dtype, S)
        budget = torch.empty(rows, dtype=torch.int64, device=dev)
        prob = torch.empty(rows, dtype=dtype, device=dev)
        stats = torch.empty((rows, 4), dtype=torch.float32, device=dev)
        table = _native_ops.exp_table(dev) if dtype == torch.bfloat16 else None
        W = words_per_row(S)
        _native.check(
            lib.sah_adaptive_budget(
                scores.data_ptr(), _native.dtype_code(dtype), float(scaling), bptr, bsb, bsh, bsq,
                _native.ptr(prev_nb.bits) if prev_nb is not None else None,
                _native.ptr(prev_nb.data) if prev_nb is not None else None,
                _native.ptr(prev_nb.wpre) if prev_nb is not None and prev_nb.data is not None else None,
                _native.ptr(prev_nb.ptr) if prev_nb is not None and prev_nb.data is not None else None,
                B, H, Sq, S, W, start, end, nb, base_seed, _native.ptr(base_draws), _native.ptr(table),
                float(self.delta_ppf), float(self.epsilon), budget.data_ptr(), prob.data_ptr(),
                stats.data_ptr(), st),
            "sah_adaptive_budget")
        del keep
        meta.setdefault("adaptive_sampling_stats", {})[layer_idx] = (budget, prob, stats)

        sptr = torch.zeros(rows + 1, dtype=torch.int64, device=dev)
        torch.cumsum(budget, dim=0, out=sptr[1:])
        samp = torch.zeros((rows, W), dtype=torch.int32, device=dev)
        _native.check(
            lib.sah_sample_scatter(sptr.data_ptr(), rows, _native.ptr(pool), base_seed + 1, start, n, S,
                                   W, _native.sm_count(dev), samp.data_ptr(), st),
            "sah_sample_scatter")
        return _native_ops.merge_sampled_bits(previous_mask, samp, prob, rows * n)

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "AdaptiveSamplingMasker":
        if not isinstance(config, AdaptiveSamplingMaskerConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
