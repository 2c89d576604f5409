"""Unscaled q.k scores in the input dtype (oracle_top_k.py:70-73,
adaptive_sampling.py:183-197 before scaling)."""

import numpy as np

from .bf16 import round_to


def qk_scores(q, k, dtype: str, attention_mask=None) -> np.ndarray:
    """`torch.matmul(queries, keys.transpose(-2, -1))` for GQA-repeated keys,
    result rounded to `dtype`, then `+ attention_mask` rounded again.

    Summation order fixed here (the reference leaves it to its BLAS): eight
    interleaved fp32 partial sums p_i = sum_t x[8t+i] * y[8t+i] with t ascending
    (product rounded to fp32, then added), combined as
    ((p0+p1)+(p2+p3)) + ((p4+p5)+(p6+p7)).
    q [B,Hq,Sq,D], k [B,Hkv,S,D] -> [B,Hq,Sq,S] float32 holding `dtype` values.
    """
    q = np.asarray(q, np.float32)
    k = np.asarray(k, np.float32)
    B, Hq, Sq, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    G = Hq // Hkv
    out = np.empty((B, Hq, Sq, S), np.float32)
    for b in range(B):
        for h in range(Hq):
            kh = k[b, h // G].reshape(S, D // 8, 8)
            for qi in range(Sq):
                qv = q[b, h, qi].reshape(D // 8, 8)
                p = np.zeros((S, 8), np.float32)
                for t in range(D // 8):
                    p = p + kh[:, t, :] * qv[t][None, :]
                s = ((p[:, 0] + p[:, 1]) + (p[:, 2] + p[:, 3])) + ((p[:, 4] + p[:, 5]) + (p[:, 6] + p[:, 7]))
                out[b, h, qi] = s
    out = round_to(out, dtype)
    if attention_mask is not None:
        out = round_to(out + np.asarray(attention_mask, np.float32)[..., :S], dtype)
    return out
