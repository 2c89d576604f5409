"""OracleTopP restated on numpy arrays.  Test infrastructure only: nothing in the package may
import this module.

Reference: research_attention/maskers/fixed/implementations/oracle_top_p.py
  _should_use_full_attention :80-83, _compute_exp_attention_scores :85-106,
  _compute_top_p_thresholds :108-136, _create_oracle_top_p_mask :138-169.

Every tensor operation of the reference is one rounding to the tensors' dtype.  What decides
the selection is the running sum of the descending-sorted weights; torch's CPU cumsum keeps
one accumulator per row (float32 for bfloat16 tensors), adds the sorted values one after the
other and rounds every prefix to the dtype.  Only bfloat16 is restated: a float32 tensor is
accumulated in float64 by the reference, over values that do not fall into a small set.
"""

import numpy as np

from . import qk, sampling
from .bf16 import bits_of, from_bits, round_bf16

BF16_MIN = np.float32(-3.3895313892515355e38)  # torch.finfo(torch.bfloat16).min


def exp_weights(scores: np.ndarray, scaling: float, attention_mask, prev_active: np.ndarray) -> np.ndarray:
    """:85-106.  scores: unscaled q.k in bf16, [B,Hq,Sq,S] float32 holding bf16 values."""
    raw = round_bf16(scores.astype(np.float32) * np.float32(scaling))
    if attention_mask is not None:
        raw = round_bf16(raw + np.asarray(attention_mask, np.float32)[..., : raw.shape[-1]])
    raw = np.where(prev_active, BF16_MIN, raw)
    mx = raw.max(axis=-1, keepdims=True)
    with np.errstate(over="ignore", invalid="ignore"):
        diff = round_bf16((raw - mx).astype(np.float32))
    return sampling.exp_dtype(diff, "bf16")


def sequential_prefix_sums(sorted_desc: np.ndarray) -> np.ndarray:
    """float32 running sums of one row in the given order, every prefix rounded to bf16.
    numpy's float32 cumsum keeps one accumulator and adds element by element, which is the
    order wanted here (`sequential_prefix_sums_loop` spells it out; a test compares the two)."""
    return round_bf16(np.cumsum(sorted_desc.astype(np.float32), dtype=np.float32))


def sequential_prefix_sums_loop(sorted_desc: np.ndarray) -> np.ndarray:
    acc = np.float32(0.0)
    out = np.empty(sorted_desc.shape[0], np.float32)
    for i, x in enumerate(sorted_desc.astype(np.float32)):
        acc = np.float32(acc + x)
        out[i] = acc
    return round_bf16(out)


def threshold_row(weights_row: np.ndarray, top_p: float) -> np.float32:
    """:108-136 for one row."""
    srt = np.sort(weights_row.astype(np.float32))[::-1]
    cums = sequential_prefix_sums(srt)
    total = cums[-1]
    with np.errstate(divide="ignore", invalid="ignore"):
        norm = round_bf16((cums / total).astype(np.float32))
    p = round_bf16(np.array([top_p], np.float32))[0]
    pos = int(np.searchsorted(norm, p, side="right"))
    pos = min(pos, srt.shape[0] - 1)
    return srt[pos]


def select(scores: np.ndarray, scaling: float, attention_mask, prev_active: np.ndarray,
           top_p: float) -> np.ndarray:
    """Boolean [B,Hq,Sq,S]: weights >= the row's threshold (:158-160)."""
    w = exp_weights(scores, scaling, attention_mask, prev_active)
    flat = w.reshape(-1, w.shape[-1])
    out = np.zeros(flat.shape, bool)
    for r in range(flat.shape[0]):
        out[r] = flat[r] >= threshold_row(flat[r], top_p)
    return out.reshape(w.shape)


def apply(prm, st, q, k, scaling, attention_mask, meta) -> None:
    """One masker step on a stacks.StackState."""
    from . import mask_ops

    S = k.shape[2]
    if st.dtype != "bf16":
        raise NotImplementedError("OracleTopP is restated for bfloat16 only")
    if S <= int(prm["top_p"] * S):  # :80-83
        st.full = True
        return
    s = meta["oracle_scores_in"] if "oracle_scores_in" in meta else qk.qk_scores(q, k, st.dtype, None)
    sel = select(np.asarray(s, np.float32), scaling, attention_mask, st.mask != 0, prm["top_p"])
    st.set(mask_ops.merge(st.mask, sel.astype(np.float32), st.dtype))
