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
            if prm.get("metric", "euclidean") == "ip":  # pq_top_k.py:233-237
                X, meta["pq_ip2l2_phi"] = pq.ip2l2_augment(X, st.dtype)
            init_idx = np.asarray(meta["pq_init_indices"])
            init = X[np.arange(X.shape[0])[:, None], init_idx]
            codes, C = pq.kmeans(X, init, prm["kmeans_iter"], meta.get("pq_reseed_indices"))
            meta["pq_centroids"] = round_to(C, st.dtype).reshape(B, Hkv, n_sub, cent, X.shape[2])
            meta["pq_codes"] = codes.reshape(B, Hkv, n_sub, n).transpose(0, 1, 3, 2)
        s = pq.scores(q, meta["pq_centroids"], meta["pq_codes"], st.dtype)
        meta["pq_scores"] = s
        full = np.zeros((B, Hq, Sq, S), np.float32)
        full[..., off:off + n] = s
        sel = topk.topk_inactive(full, st.mask != 0, heavy, off, off + n)
        st.set(mask_ops.merge(st.mask, sel.astype(np.float32), st.dtype))
    elif kind == "magicpig":
        from . import magicpig
        magicpig.apply(prm, st, q, k, meta)
    elif kind in ("random_sampling", "adaptive_sampling"):
        _apply_sampling(kind, prm, st, q, k, v, scaling, attention_mask, meta)
    elif kind == "quest_topk":
        from . import quest
        quest.apply(prm, st, q, k, attention_mask, meta)
    elif kind == "oracle_topp":
        from . import topp
        topp.apply(prm, st, q, k, scaling, attention_mask, meta)
    else:
        raise ValueError(f"unknown masker kind {kind}")


def _apply_sampling(kind, prm, st, q, k, v, scaling, attention_mask, meta) -> None:
    from scipy.stats import norm

    from . import qk, sampling

    B, Hq, Sq, _ = q.shape
    S = k.shape[2]
    rows = B * Hq * Sq
    if kind == "random_sampling":
        n = int(prm["sampling_rate"] * S)
        draws = np.asarray(meta["random_sampling_draws"]).reshape(rows, n)
        dense = np.zeros((rows, S), np.float32)
        p = round_to(np.float32(prm["sampling_rate"]), st.dtype)
        for r in range(rows):
            dense[r, draws[r]] = p
        st.set(mask_ops.merge(st.mask, dense.reshape(st.mask.shape), st.dtype))
        return
    # adaptive sampling
    if prm["base_rate_sampling"] == 0:
        return
    start, end, n = sampling.sampling_range(S, prm["init_offset"], prm["local_offset"])
    if n < 2:
        st.full = True
        return
    nb = sampling.base_count(prm["base_rate_sampling"], n)
    scores = meta.get("oracle_scores_unbiased")
    if scores is None:
        scores = qk.qk_scores(q, k, st.dtype, None)
    seed = int(meta.get("adaptive_seed", 0))
    base = meta.get("adaptive_base_draws")
    if base is None:
        base = sampling.draw_columns(seed, np.arange(rows * nb, dtype=np.uint64), start, n)
    base = np.asarray(base).reshape(rows, nb)
    ppf = float(norm.ppf(1 - prm["delta"]))
    prev = None if st.empty else st.mask.reshape(rows, S)
    bias = None
    if attention_mask is not None:
        bias = np.broadcast_to(np.asarray(attention_mask, np.float32)[..., :S], (B, Hq, Sq, S)).reshape(rows, S)
    budgets, probs, stats = [], [], []
    sc = scores.reshape(rows, S)
    for r in range(rows):
        bgt, p, stt = sampling.adaptive_budget_row(
            sc[r], scaling, None if bias is None else bias[r], None if prev is None else prev[r],
            start, end, nb, base[r], ppf, prm["epsilon"], st.dtype)
        budgets.append(bgt)
        probs.append(p)
        stats.append(stt)
    meta["adaptive_budget"] = np.array(budgets, np.int64)
    meta["adaptive_prob"] = np.array(probs, np.float32)
    meta["adaptive_stats"] = np.array(stats, np.float32)
    total = int(sum(budgets))
    pool = meta.get("adaptive_pool")
    if pool is None:
        pool = sampling.draw_columns(seed + 1, np.arange(total, dtype=np.uint64), start, n)
    pool = np.asarray(pool)[:total]
    dense = np.zeros((rows, S), np.float32)
    pos = 0
    for r in range(rows):
        dense[r, pool[pos:pos + budgets[r]]] = probs[r]
        pos += budgets[r]
    st.set(mask_ops.merge(st.mask, dense.reshape(st.mask.shape), st.dtype))

