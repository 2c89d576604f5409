"""PQCache restated: batched k-means, code lookup scores
(research_attention/maskers/fixed/implementations/pq_top_k.py, utils/pq_utils.py)."""

import numpy as np

from .bf16 import round_to


def _sq_dist(X: np.ndarray, C: np.ndarray, dtype_math: str = None) -> np.ndarray:
    """[g,n,d] x [g,k,d] -> [g,n,k]: sum over ascending dims of (x - c)^2 in fp32
    (pairwise_distance_batched, pq_utils.py:246-255).  With `dtype_math` every
    operation is rounded to that dtype (quantisation of appended keys, pq_top_k.py:388-404)."""
    g, n, d = X.shape
    acc = np.zeros((g, n, C.shape[1]), np.float32)
    for j in range(d):
        t = X[:, :, None, j] - C[:, None, :, j]
        if dtype_math:
            t = round_to(t, dtype_math)
            acc = acc + round_to(t * t, dtype_math)
        else:
            acc = acc + t * t
    return round_to(acc, dtype_math) if dtype_math else acc


def assign(X: np.ndarray, C: np.ndarray, chunk: int = 256, dtype_math: str = None) -> np.ndarray:
    """argmin over centroids, first minimum wins (torch.argmin)."""
    out = np.empty(X.shape[:2], np.int64)
    for s in range(0, X.shape[1], chunk):
        out[:, s:s + chunk] = np.argmin(_sq_dist(X[:, s:s + chunk], C, dtype_math), axis=2)
    return out


def kmeans(X: np.ndarray, init_centers: np.ndarray, iter_limit: int, reseed=None, tol: float = 1e-4):
    """kmeans_batched (pq_utils.py:260-438) with caller-given initial centres.

    Per iteration: assignment, centre = fp32(sum) / fp32(count) with the sums taken in
    float64 (order independent), empty clusters take key `reseed[it][g, c]`, stop when
    every group's (sum of centre moves)^2 < tol or after `iter_limit` iterations.
    Returns (codes of the last assignment, centres after the last update)."""
    X = np.asarray(X, np.float32)
    C = np.asarray(init_centers, np.float32).copy()
    g, n, d = X.shape
    k = C.shape[1]
    it = 0
    while True:
        codes = assign(X, C)
        sums = np.zeros((g, k, d), np.float64)
        counts = np.zeros((g, k), np.int64)
        for gi in range(g):
            np.add.at(sums[gi], codes[gi], X[gi].astype(np.float64))
            counts[gi] = np.bincount(codes[gi], minlength=k)
        new = sums.astype(np.float32) / np.maximum(counts, 1).astype(np.float32)[..., None]
        empty = counts == 0
        if empty.any():
            if reseed is None:
                raise ValueError("empty cluster and no reseed indices")
            rs = np.asarray(reseed[it])
            new = np.where(empty[..., None], X[np.arange(g)[:, None], rs], new)
        diff = new - C
        move = np.zeros((g, k), np.float32)
        for j in range(d):
            move = move + diff[..., j] * diff[..., j]
        shift = np.sqrt(move).sum(axis=1, dtype=np.float32)
        C = new.astype(np.float32)
        it += 1
        if np.all(shift * shift < np.float32(tol)) or (iter_limit and it >= iter_limit):
            break
    return codes, C


def split_keys(k: np.ndarray, init_offset: int, n_sub: int) -> np.ndarray:
    """[B,Hkv,S,D] -> [B*Hkv*n_sub, S-init_offset, D/n_sub] (pq_top_k.py:214-231)."""
    B, Hkv, S, D = k.shape
    sd = D // n_sub
    x = k[:, :, init_offset:].reshape(B, Hkv, S - init_offset, n_sub, sd).transpose(0, 1, 3, 2, 4)
    return np.ascontiguousarray(x).reshape(B * Hkv * n_sub, S - init_offset, sd)


def ip2l2_augment(X: np.ndarray, dtype: str):
    """ip2l2_augment (utils/pq_utils.py:585-612) on dtype values: [g,n,d] -> ([g,n,d+1], phi [g,1,1]).
    Every tensor operation of the reference is one rounding to the dtype: x**2, the sum over the
    sub-vector (float32 accumulator, rounded once), phi - |x|^2, the square root."""
    X = np.asarray(X, np.float32)
    sq = round_to(X * X, dtype)
    acc = np.zeros(X.shape[:2], np.float32)
    for j in range(X.shape[2]):
        acc = acc + sq[:, :, j]
    norms_sq = round_to(acc, dtype)[..., None]
    phi = norms_sq.max(axis=1, keepdims=True)
    extra = round_to(np.sqrt(round_to(phi - norms_sq, dtype)), dtype)
    return np.concatenate([X, extra], axis=2).astype(np.float32), phi


def scores(q, centroids, codes, dtype: str) -> np.ndarray:
    """_compute_pq_scores (pq_top_k.py:406-490).
    q [B,Hq,Sq,D]; centroids [B,Hkv,n_sub,cent,sd] (dtype values; with metric "ip" they carry one
    more column, which scoring leaves out, pq_top_k.py:443-458); codes [B,Hkv,n,n_sub].
    lut = q_sub . centroid (fma over ascending dims, rounded to dtype); score = fp32 sum of
    the table entries over ascending sub-vectors, rounded once.  -> [B,Hq,Sq,n]"""
    q = np.asarray(q, np.float32)
    B, Hq, Sq, D = q.shape
    _, Hkv, n_sub, cent, _ = centroids.shape
    sd = D // n_sub
    G = Hq // Hkv
    n = codes.shape[2]
    out = np.empty((B, Hq, Sq, n), np.float32)
    for b in range(B):
        for h in range(Hq):
            kv = h // G
            for qi in range(Sq):
                qs = q[b, h, qi].reshape(n_sub, sd)
                acc = np.zeros((n_sub, cent), np.float32)
                for d in range(sd):
                    acc = (acc.astype(np.float64)
                           + qs[:, d:d + 1].astype(np.float64) * centroids[b, kv, :, :, d].astype(np.float64)
                           ).astype(np.float32)
                lut = round_to(acc, dtype)
                s = np.zeros(n, np.float32)
                for sub in range(n_sub):
                    s = s + lut[sub, codes[b, kv, :, sub]]
                out[b, h, qi] = s
    return round_to(out, dtype)
