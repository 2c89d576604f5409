"""Quest page top-k restated on numpy arrays.  Test infrastructure only: nothing in the package
may import this module.

Reference: research_attention/maskers/fixed/implementations/quest_top_k.py (add_mask :72-106,
_create_quest_page_topk_mask :108-196, full-attention rule :198-202) and utils/quest_utils.py
(compute_page_min_max :10-50, quest_page_scores :53-67, pages_to_token_mask :70-93,
attention_mask_to_allowed_prob :96-112, pages_valid :115-137).  label_bits = 16 only (no
pseudo-quantisation of the page bounds).

The page score is sum_j max(q_j * min_j, q_j * max_j) with every product rounded to the
tensors' dtype and the sum taken by torch's CPU row reduction: float32 accumulation in vectors
of 8 lanes (a bfloat16 load brings 16 elements and adds its two halves), four interleaved vector
accumulators added in order, then the 8 lanes added in order (`row_sum`).
"""

import numpy as np

from . import mask_ops, topk
from .bf16 import round_to

F32 = np.float32
FINFO_MIN = {"bf16": F32(-3.3895313892515355e38), "f32": np.finfo(np.float32).min}


def row_sum(m: np.ndarray, dtype: str) -> np.ndarray:
    """Sum over the last axis in torch's CPU order (vectorized_inner_sum / row_sum /
    multi_row_sum of ATen's SumKernel, 8-lane float vectors), rounded to `dtype`."""
    lanes = 8
    a = m.reshape(-1, m.shape[-1]).astype(F32)
    n, D = a.shape
    vec = 2 * lanes if dtype == "bf16" else lanes
    nv = D // vec
    if dtype == "bf16":
        loads = [(a[:, i * vec:i * vec + lanes] + a[:, i * vec + lanes:(i + 1) * vec]).astype(F32) for i in range(nv)]
    else:
        loads = [a[:, i * vec:(i + 1) * vec] for i in range(nv)]
    ilp = 4
    full = nv // ilp
    acc = [np.zeros((n, lanes), F32) for _ in range(ilp)]
    for i in range(full):
        for k in range(ilp):
            acc[k] = (acc[k] + loads[i * ilp + k]).astype(F32)
    for i in range(full * ilp, nv):
        acc[0] = (acc[0] + loads[i]).astype(F32)
    for k in range(1, ilp):
        acc[0] = (acc[0] + acc[k]).astype(F32)
    fin = np.zeros(n, F32)
    for j in range(nv * vec, D):
        fin = (fin + a[:, j]).astype(F32)
    for lane in range(lanes):
        fin = (fin + acc[0][:, lane]).astype(F32)
    return round_to(fin, dtype).reshape(m.shape[:-1])


def page_min_max(k: np.ndarray, page_size: int):
    """[B,Hkv,S,D] -> (min, max) [B,Hkv,P,D]; the last page may be partial (:10-50)."""
    B, H, S, D = k.shape
    P = -(-S // page_size)
    pmin = np.empty((B, H, P, D), F32)
    pmax = np.empty((B, H, P, D), F32)
    for p in range(P):
        blk = k[:, :, p * page_size:min(S, (p + 1) * page_size), :]
        pmin[:, :, p], pmax[:, :, p] = blk.min(axis=2), blk.max(axis=2)
    return pmin, pmax


def page_scores(q: np.ndarray, pmin: np.ndarray, pmax: np.ndarray, dtype: str) -> np.ndarray:
    """q [B,Hq,Sq,D], bounds [B,Hkv,P,D] -> [B,Hq,Sq,P] (:53-67)."""
    G = q.shape[1] // pmin.shape[1]
    lo = np.repeat(pmin, G, axis=1)[:, :, None, :, :]
    hi = np.repeat(pmax, G, axis=1)[:, :, None, :, :]
    qq = q.astype(F32)[:, :, :, None, :]
    m = np.maximum(round_to(qq * lo, dtype), round_to(qq * hi, dtype))
    return row_sum(m, dtype)


def apply(prm, st, q, k, attention_mask, meta) -> None:
    """One masker step on a stacks.StackState."""
    B, Hq, Sq, D = q.shape
    S = k.shape[2]
    if prm.get("label_bits", 16) != 16:
        raise NotImplementedError("label_bits < 16 is not restated")
    heavy = mask_ops.effective_size(prm["heavy_size"], S)
    if S <= max(1, heavy):  # :198-202
        st.full = True
        return
    ps = int(prm["page_size"])
    P = -(-S // ps)
    pmin, pmax = page_min_max(np.asarray(k, F32), ps)
    sc = page_scores(np.asarray(q, F32), pmin, pmax, st.dtype)
    allowed = None
    if attention_mask is not None:  # :96-137, :156-170
        allowed = (np.asarray(attention_mask, F32)[..., :S] >= 0)
        pad = np.zeros(allowed.shape[:-1] + (P * ps,), bool)
        pad[..., :S] = allowed
        valid = pad.reshape(allowed.shape[:-1] + (P, ps)).any(-1)            # [B,1,Sq|1,P]
        sc = np.where(np.broadcast_to(valid, sc.shape), sc, FINFO_MIN[st.dtype])
    meta["quest_page_scores"] = sc
    kp = min(P, max(3, heavy // ps))
    if kp <= 0:
        kp = 1
    sel_pages = topk.topk_inactive(sc, np.zeros(sc.shape, bool), kp)          # [B,Hq,Sq,P]
    union = np.repeat(sel_pages, ps, axis=-1)[..., :S].astype(F32)
    dense = np.maximum(np.clip(st.mask, 0.0, 1.0), union)
    if allowed is not None:
        dense = dense * np.broadcast_to(allowed, dense.shape).astype(F32)
    st.set(round_to(dense.astype(F32), st.dtype))
