"""Masker stacks end to end: ResearchAttention.custom_attention
(research_attention/base.py:63-170) restated on numpy arrays.

A stack is a list of (kind, params) pairs applied in order to a dense mask
that starts empty; the result goes through `attention.masked_attention`.
"""

from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import attention, hashattention, mask_ops, qk, topk


class StackState:
    """What the reference keeps between maskers: the dense mask and the full/empty flags."""

    def __init__(self, shape, dtype: str):
        self.mask = np.zeros(shape, np.float32)
        self.full = False
        self.empty = True
        self.dtype = dtype

    def set(self, mask: np.ndarray) -> None:
        self.mask, self.empty = mask, False


def apply_masker(kind: str, prm: Dict[str, Any], st: StackState, q, k, v, scaling,
                 attention_mask, meta: Dict[str, Any]) -> None:
    if st.full:  # every masker returns a full previous mask unchanged
        return
    B, Hq, Sq, _ = q.shape
    S = k.shape[2]
    if kind == "sink":
        n = mask_ops.effective_size(prm["sink_size"], S)
        if S <= n:  # basic_fixed.py:424-428
            st.full = True
            return
        st.set(mask_ops.sink(st.mask, n))
    elif kind == "local":
        w = mask_ops.effective_size(prm["window_size"], S)
        if S <= w + Sq:  # basic_fixed.py:220-224
            st.full = True
            return
        st.set(mask_ops.local(st.mask, w))
    elif kind == "oracle_topk":
        kk = mask_ops.effective_size(prm["heavy_size"], S)
        if S <= kk:
            st.full = True
            return
        if "oracle_scores_in" in meta:  # scores handed in by a test
            s = np.asarray(meta["oracle_scores_in"], np.float32)
        else:
            s = qk.qk_scores(q, k, st.dtype, attention_mask)
        meta["oracle_scores"] = s
        sel = topk.topk_inactive(s, st.mask != 0, kk)
        out = st.mask.copy()
        out[sel] = 1.0  # scatter_(1.0) into the previous dense mask (oracle_top_k.py:79)
        st.set(out)
    elif kind == "hash_topk":
        kk = mask_ops.effective_size(prm["heavy_size"], S)
        if S <= kk:
            st.full = True
            return
        G = Hq // k.shape[1]
        w = prm["weights"]
        if "hash_kcodes" not in meta:  # keys repeated, then hashed per query head (:354-359)
            meta["hash_kcodes"] = hashattention.signatures(
                attention.repeat_kv(k, G), w["key_matrix"], w["key_bias"], prm["activation"], st.dtype)
        if "hash_qcodes_in" in meta:  # codes handed in by a test
            meta["hash_qcodes"] = meta["hash_qcodes_in"]
        else:
            meta["hash_qcodes"] = hashattention.signatures(q, w["query_matrix"], w["query_bias"],
                                                           prm["activation"], st.dtype)
        s = hashattention.scores(meta["hash_qcodes"], meta["hash_kcodes"], prm["bits"], st.dtype,
                                 attention_mask)
        meta["hash_scores"] = s
        sel = topk.topk_inactive(s, st.mask != 0, kk)
        st.set(mask_ops.merge(st.mask, sel.astype(np.float32), st.dtype))
    else:
        from . import extra_maskers  # adaptive sampling, MagicPig, PQCache
        extra_maskers.apply(kind, prm, st, q, k, v, scaling, attention_mask, meta)


def run_stack(stack: List[Tuple[str, Dict[str, Any]]], q, k, v, scaling: float, dtype: str,
              attention_mask=None, sinks=None, meta: Optional[Dict[str, Any]] = None):
    """Returns (dense mask or None when full/empty, output [B,Sq,Hq,D], meta)."""
    meta = {} if meta is None else meta
    B, Hq, Sq, _ = q.shape
    st = StackState((B, Hq, Sq, k.shape[2]), dtype)
    for kind, prm in stack:
        apply_masker(kind, prm, st, q, k, v, scaling, attention_mask, meta)
    no_mask = st.full or st.empty
    out = attention.masked_attention(q, k, v, None if no_mask else st.mask, scaling, dtype,
                                     attention_mask, sinks, no_mask=no_mask)
    meta["full"], meta["empty"] = st.full, st.empty
    return (None if no_mask else st.mask), out, meta
