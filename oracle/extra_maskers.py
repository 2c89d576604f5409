"""Maskers beyond sink / local / oracle top-k / hash top-k, dispatched from stacks.apply_masker."""

import numpy as np

from . import mask_ops, pq, topk
from .bf16 import round_to


def apply(kind, prm, st, q, k, v, scaling, attention_mask, meta) -> None:
    B, Hq, Sq, _ = q.shape
    S = k.shape[2]
    if kind == "pq_topk":
        heavy = mask_ops.effective_size(prm["heavy_size"], S)
        off, n_sub, bits = prm["init_offset"], prm["pq_group_factor"], prm["pq_bits"]
        if S <= heavy + off + Sq + 2 ** bits:  # pq_top_k.py:167-174
            st.full = True
            return
        Hkv, D = k.shape[1], k.shape[3]
        n, cent, sd = S - off, 2 ** bits, D // n_sub
        if "pq_centroids" not in meta:
            X = pq.split_keys(k, off, n_sub)
            init_idx = np.asarray(meta["pq_init_indices"])
            init = X[np.arange(X.shape[0])[:, None], init_idx]
            codes, C = pq.kmeans(X, init, prm["kmeans_iter"], meta.get("pq_reseed_indices"))
            meta["pq_centroids"] = round_to(C, st.dtype).reshape(B, Hkv, n_sub, cent, sd)
            meta["pq_codes"] = codes.reshape(B, Hkv, n_sub, n).transpose(0, 1, 3, 2)
        s = pq.scores(q, meta["pq_centroids"], meta["pq_codes"], st.dtype)
        meta["pq_scores"] = s
        full = np.zeros((B, Hq, Sq, S), np.float32)
        full[..., off:off + n] = s
        sel = topk.topk_inactive(full, st.mask != 0, heavy, off, off + n)
        st.set(mask_ops.merge(st.mask, sel.astype(np.float32), st.dtype))
    else:
        raise ValueError(f"unknown masker kind {kind}")
