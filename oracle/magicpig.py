"""MagicPig restated (research_attention/maskers/sampling/implementations/magic_pig.py).

Every tensor operation of the reference is one rounding to the dtype; reductions over the
head dimension use "lane order": channel c belongs to lane c // (D/32), a lane sums its
channels in ascending order, the 32 lane sums combine by an xor tree (16, 8, 4, 2, 1).
Projections accumulate over channels in ascending order in one float32 accumulator.
"""

import numpy as np

from . import mask_ops
from .bf16 import bits_of, from_bits, round_bf16, round_to

F = np.float32


def lane_sum(x: np.ndarray) -> np.ndarray:
    """Sum over the last axis (length a multiple of 32) in lane order, float32."""
    x = np.asarray(x, F)
    D = x.shape[-1]
    per = D // 32
    lanes = x.reshape(x.shape[:-1] + (32, per))
    acc = np.zeros(x.shape[:-1] + (32,), F)
    for t in range(per):
        acc = acc + lanes[..., t]
    idx = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        acc = acc + acc[..., idx ^ off]
    return acc[..., 0]


def key_mean(k: np.ndarray, dtype: str, shard=None) -> np.ndarray:
    """keys.mean(dim=2) (:175-176): float64 sum / S, rounded through float32 to the dtype.
    With a sequence shard the sum runs over all ranks and S is the whole length."""
    s = np.asarray(k, np.float64).sum(axis=2)
    n = k.shape[2]
    if shard is not None:
        s, n = shard.comm.all_reduce_sum(s), shard.total
    return round_to((s / n).astype(F), dtype)  # [B,Hkv,D]


def centred(x: np.ndarray, mean, dtype: str) -> np.ndarray:
    return np.asarray(x, F) if mean is None else round_to(np.asarray(x, F) - mean, dtype)


def norms(c: np.ndarray, dtype: str) -> np.ndarray:
    return round_to(np.sqrt(lane_sum(c * c)), dtype)


def augment(nk: np.ndarray, M, dtype: str) -> np.ndarray:
    r = lambda v: round_to(np.asarray(v, F), dtype)  # noqa: E731
    M = F(M)
    d = r(r(M * M) - r(nk * nk))
    return r(r(np.sqrt(d)) / M)


def project_signs(x: np.ndarray, proj: np.ndarray) -> np.ndarray:
    """x [n, D+1] float32, proj [D+1, bits] -> bool [n, bits]: projection > 0."""
    acc = np.zeros((x.shape[0], proj.shape[1]), F)
    with np.errstate(invalid="ignore"):
        for c in range(x.shape[1]):
            acc = acc + x[:, c:c + 1] * proj[c][None, :].astype(F)
    return acc > 0


def pack(signs: np.ndarray, L: int, K: int) -> np.ndarray:
    """bool [n, L*K] -> int64 [n, L]; bit j of table l is column l*K + j (:120-150)."""
    w = (1 << np.arange(K, dtype=np.int64))
    return (signs.reshape(-1, L, K).astype(np.int64) * w).sum(-1)


def key_codes(k_shard: np.ndarray, mean, nk: np.ndarray, M, proj: np.ndarray, L: int, K: int,
              dtype: str) -> np.ndarray:
    """k_shard [B,Hkv,n,D] -> codes int64 [B,Hkv,n,L] with the maximum norm M."""
    B, Hkv, n, D = k_shard.shape
    c = centred(k_shard, None if mean is None else mean[:, :, None, :], dtype)
    ks = round_to(c / F(M), dtype)
    aug = augment(nk, M, dtype)
    x = np.concatenate([ks, aug[..., None]], axis=-1).reshape(-1, D + 1)
    return pack(project_signs(x, proj), L, K).reshape(B, Hkv, n, L)


_TABLES = {}


def prob_table(K: int, L: int) -> np.ndarray:
    """uint16[65536]: bf16 bits of the cosine -> bf16 bits of 1 - (1 - (1 - acos(c)/pi)^K)^L,
    each step rounded to bf16 (:389-403)."""
    if (K, L) not in _TABLES:
        bf = lambda v: round_bf16(np.asarray(v, np.float64).astype(F)).astype(np.float64)  # noqa: E731
        with np.errstate(invalid="ignore", over="ignore"):
            c = from_bits(np.arange(65536, dtype=np.uint32).astype(np.uint16)).astype(np.float64)
            c = np.clip(c, -1.0, 1.0)
            theta = bf(np.arccos(c))
            a = bf((theta.astype(F) / F(np.pi)).astype(np.float64))
            s = bf(1.0 - a)
            st = bf(np.power(s, float(K)))
            u = bf(1.0 - st)
            ul = bf(np.power(u, float(L)))
            p = round_bf16((1.0 - ul).astype(F))
        t = bits_of(p)
        t[np.isnan(p)] = 0x7FC0
        _TABLES[(K, L)] = t
    return _TABLES[(K, L)]


def collision_prob(c: np.ndarray, K: int, L: int, dtype: str) -> np.ndarray:
    c = np.clip(np.asarray(c, F), F(-1), F(1))
    if dtype == "bf16":
        return from_bits(prob_table(K, L)[bits_of(c)])
    theta = np.arccos(c.astype(np.float64)).astype(F)
    a = theta / F(np.pi)
    s = F(1) - a
    st = np.power(s.astype(np.float64), float(K)).astype(F)
    u = F(1) - st
    ul = np.power(u.astype(np.float64), float(L)).astype(F)
    return (F(1) - ul).astype(F)


def apply(prm, st, q, k, meta, shard=None) -> None:
    """One MagicPig.add_mask (:510-593) on the stack state.  `shard` (begin, total, comm):
    `k` is one rank's key range; the key mean and the maximum key norm are global."""
    dtype = st.dtype
    r = lambda v: round_to(np.asarray(v, F), dtype)  # noqa: E731
    B, Hq, Sq, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    G = Hq // Hkv
    L, K = prm["lsh_l"], prm["lsh_k"]
    proj = np.asarray(meta["lsh_projection"], F)
    mean = None
    if prm.get("center", True):
        if meta.get("lsh_key_mean") is None:
            meta["lsh_key_mean"] = key_mean(k, dtype, shard)
        mean = meta["lsh_key_mean"]
    # key state: norms of all keys seen, running maximum, codes computed with the maximum of
    # the call that first saw each key
    state = meta.setdefault("lsh_state", {"codes": np.zeros((B, Hkv, 0, L), np.int64),
                                          "norms": np.zeros((B, Hkv, 0), F), "M": F(0)})
    n0 = state["codes"].shape[2]
    if state["norms"].shape[2] < n0:  # codes handed in without norms
        c_old = centred(k[:, :, :n0], None if mean is None else mean[:, :, None, :], dtype)
        state["norms"] = norms(c_old, dtype)
        state["M"] = F(max(state["M"], state["norms"].max()))
    if S > n0:
        c_new = centred(k[:, :, n0:], None if mean is None else mean[:, :, None, :], dtype)
        nk_new = norms(c_new, dtype)
        state["M"] = F(max(state["M"], nk_new.max()))
        if shard is not None:
            state["M"] = F(shard.comm.all_reduce_max(np.array([state["M"]], F))[0])
        codes_new = key_codes(k[:, :, n0:], mean, nk_new, state["M"], proj, L, K, dtype)
        state["codes"] = np.concatenate([state["codes"], codes_new], axis=2)
        state["norms"] = np.concatenate([state["norms"], nk_new], axis=2)
    M = state["M"]
    meta["lsh_key_codes"] = state["codes"]

    # queries
    qmean = None if mean is None else np.repeat(mean, G, axis=1)[:, :, None, :]
    qc = centred(q, qmean, dtype)
    qn = r(qc / r(norms(qc, dtype) + F(1e-8))[..., None])
    xq = np.concatenate([qn, np.zeros(qn.shape[:-1] + (1,), F)], axis=-1).reshape(-1, D + 1)
    qcodes = pack(project_signs(xq, proj), L, K).reshape(B, Hq, Sq, L)
    if "lsh_query_codes_in" in meta:  # codes handed in by a test
        qcodes = np.asarray(meta["lsh_query_codes_in"]).reshape(B, Hq, Sq, L)
    meta["lsh_query_codes"] = qcodes
    qunit = r(qn / r(norms(qn, dtype) + F(1e-8))[..., None])

    kcodes = np.repeat(state["codes"], G, axis=1)  # [B,Hq,S,L]
    match = (qcodes[:, :, :, None, :] == kcodes[:, :, None, :, :]).any(-1)  # [B,Hq,Sq,S]
    meta["lsh_match"] = match

    # probabilities of matched keys
    c_all = centred(k, None if mean is None else mean[:, :, None, :], dtype)
    ks = round_to(c_all / M, dtype)
    aug = augment(state["norms"], M, dtype)
    n2 = lane_sum(ks * ks) + aug * aug
    den = r(r(np.sqrt(n2)) + F(1e-8))
    kn = r(ks / den[..., None])  # [B,Hkv,S,D]
    dense = np.zeros((B, Hq, Sq, S), F)
    for b in range(B):
        for h in range(Hq):
            for i in range(Sq):
                cols = np.nonzero(match[b, h, i])[0]
                if cols.size == 0:
                    continue
                cosv = r(lane_sum(qunit[b, h, i][None, :] * kn[b, h // G, cols]))
                dense[b, h, i, cols] = collision_prob(cosv, K, L, dtype)
    meta["lsh_dense"] = dense
    st.set(mask_ops.merge(st.mask, dense, dtype))
