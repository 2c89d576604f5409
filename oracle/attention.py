"""Masked attention (sparse_attention/utils/mask_attention_utils.py:187-240, :357-491)."""

import numpy as np

from .bf16 import round_to
from .mask_ops import inv_weights


def repeat_kv(x: np.ndarray, n_rep: int) -> np.ndarray:
    """utils/kv_utils.py:5-20."""
    return x if n_rep == 1 else np.repeat(x, n_rep, axis=1)


def masked_attention(q, k, v, mask, scaling, dtype, attention_mask=None, sinks=None,
                     no_mask: bool = False, return_partials: bool = False):
    """get_masked_attention_output: fp32 dense logits over all keys, row max over
    all keys, exp, inverse mask weights, numerator / denominator, optional sink
    logit; output [B, Sq, Hq, D] rounded to `dtype`.

    q [B,Hq,Sq,D], k/v [B,Hkv,S,D], mask dense [B,Hq,Sq,S] (float32 holding
    `dtype` values) or None / no_mask=True for a full or empty Mask, which the
    reference treats as "no weights" (utils/mask.py:733-735).
    """
    q = np.asarray(q, np.float32)
    G = q.shape[1] // k.shape[1]
    kk = repeat_kv(np.asarray(k, np.float32), G)
    vv = repeat_kv(np.asarray(v, np.float32), G)
    logits = np.matmul(q, kk.transpose(0, 1, 3, 2)) * np.float32(scaling)
    if attention_mask is not None:
        logits = logits + np.asarray(attention_mask, np.float32)[..., : kk.shape[2]]
    old_max = logits.max(axis=-1, keepdims=True)
    e = np.exp(logits - old_max)
    if mask is not None and not no_mask:
        e = e * inv_weights(mask, dtype)
    num = np.matmul(e, vv)
    den = e.sum(axis=-1, keepdims=True)
    if return_partials:
        return num, den, old_max
    if sinks is not None:
        s = np.asarray(sinks, np.float32).reshape(1, -1, 1, 1)
        new_max = np.maximum(old_max, s)
        scale = np.exp(old_max - new_max)
        num, den = num * scale, den * scale + np.exp(s - new_max)
    out = round_to((num / den).astype(np.float32), dtype)
    return np.ascontiguousarray(out.transpose(0, 2, 1, 3))
