"""Top-k over inactive positions with the tie rule made explicit.

Reference: TopKMasker._get_topk_indices_from_inactive_positions
(research_attention/maskers/fixed/base.py:74-85): positions active in the
previous mask get -inf, then `torch.topk(k)`.  torch leaves the order among
equal scores unspecified; here (and in the CUDA select) the lowest column wins.
"""

import numpy as np


def topk_inactive(scores: np.ndarray, prev_active: np.ndarray, k: int,
                  col_begin: int = 0, col_end: int = None) -> np.ndarray:
    """Boolean [..., S] selection of the k best inactive columns of every row.

    Only columns in [col_begin, col_end) compete.  With fewer than k
    candidates all of them are selected.
    """
    S = scores.shape[-1]
    col_end = S if col_end is None else col_end
    flat = np.asarray(scores, dtype=np.float32).reshape(-1, S)
    act = np.asarray(prev_active, dtype=bool).reshape(-1, S)
    out = np.zeros_like(act)
    window = np.zeros(S, dtype=bool)
    window[col_begin:col_end] = True
    for r in range(flat.shape[0]):
        cand = np.flatnonzero(window & ~act[r])
        if cand.size <= k:
            out[r, cand] = True
            continue
        s = flat[r, cand] + np.float32(0.0)  # -0.0 ranks with +0.0
        order = np.argsort(-s, kind="stable")  # descending score, ascending column among ties
        out[r, cand[order[:k]]] = True
    return out.reshape(prev_active.shape)
