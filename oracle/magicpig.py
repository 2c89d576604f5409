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


def project_signs_fast(x: np.ndarray, proj: np.ndarray) -> np.ndarray:
    """`project_signs` for many rows: the signs of a float32 BLAS product, with every sum that
    a different summation order could have pushed across zero recomputed in the fixed order.

    Any float32 summation order of n products differs from the exact sum by at most
    n * 2^-24 * sum |x_c p_c| (to first order), so two orders differ by at most twice that; sums
    further from zero than 4 * n * 2^-24 * sum |x_c p_c| have the same sign in every order."""
    x = np.ascontiguousarray(x, F)
    p = np.ascontiguousarray(proj, F)
    with np.errstate(invalid="ignore"):
        acc = x @ p
        bound = (np.abs(x) @ np.abs(p)) * F(4.0 * x.shape[1] * 2.0 ** -24)
        out = acc > 0
        np.abs(acc, out=acc)
        rows, cols = np.nonzero(acc <= bound)  # a NaN sum is "not positive" in every order
        if rows.size:
            a = np.zeros(rows.size, F)
            for c in range(x.shape[1]):
                a = a + x[rows, c] * p[c, cols]
            out[rows, cols] = a > 0
    return out


def pack(signs: np.ndarray, L: int, K: int) -> np.ndarray:
    """bool [n, L*K] -> int64 [n, L]; bit j of table l is column l*K + j (:120-150)."""
    if K <= 8:  # one byte per table: the little-endian bit packing is the same weighting
        bits = np.packbits(signs.reshape(-1, L, K), axis=-1, bitorder="little")[..., 0]
        return bits.astype(np.int64)
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
    signs = project_signs(x, proj) if x.shape[0] * proj.shape[1] < (1 << 24) else project_signs_fast(x, proj)
    return pack(signs, L, K).reshape(B, Hkv, n, L)


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


def query_side(q, mean, G: int, proj, L: int, K: int, dtype: str, codes_in=None):
    """Centred, normalised queries: their table codes [B,Hq,Sq,L] and the unit vector of the
    transformed query [B,Hq,Sq,D] (:152-183, :332-372, :132-150)."""
    r = lambda v: round_to(np.asarray(v, F), dtype)  # noqa: E731
    B, Hq, Sq, D = q.shape
    qmean = None if mean is None else np.repeat(mean, G, axis=1)[:, :, None, :]
    qc = centred(q, qmean, dtype)
    qn = r(qc / r(norms(qc, dtype) + F(1e-8))[..., None])
    xq = np.concatenate([qn, np.zeros(qn.shape[:-1] + (1,), F)], axis=-1).reshape(-1, D + 1)
    qcodes = pack(project_signs(xq, proj), L, K).reshape(B, Hq, Sq, L)
    if codes_in is not None:  # codes handed in by a test
        qcodes = np.asarray(codes_in).reshape(B, Hq, Sq, L)
    qunit = r(qn / r(norms(qn, dtype) + F(1e-8))[..., None])
    return qcodes, qunit


def match_probabilities(qcodes, qunit, codes, k, mean, nk, M, K: int, L: int, dtype: str, match=None):
    """(match bool [B,Hq,Sq,n], dense float32 [B,Hq,Sq,n]) for keys `k` [B,Hkv,n,D] with table
    codes `codes` [B,Hkv,n,L] and centred norms `nk`: a key matches when any table code equals
    the query's (:455-463); matched keys carry the collision probability (:374-403, :581).
    A caller that already knows the matches passes them (`match`; `codes` is then unused)."""
    r = lambda v: round_to(np.asarray(v, F), dtype)  # noqa: E731
    B, Hq, Sq, _ = qcodes.shape
    Hkv, S = k.shape[1], k.shape[2]
    G = Hq // Hkv
    if match is None:
        match = np.zeros((B, Hq, Sq, S), bool)
        for h in range(Hq):  # one head at a time bounds the [Sq, n, L] temporary
            match[:, h] = (qcodes[:, h, :, None, :] == codes[:, h // G, None, :, :]).any(-1)
    c_all = centred(k, None if mean is None else mean[:, :, None, :], dtype)
    ks = round_to(c_all / F(M), dtype)
    aug = augment(nk, M, dtype)
    n2 = lane_sum(ks * ks) + aug * aug
    den = r(r(np.sqrt(n2)) + F(1e-8))
    kn = r(ks / den[..., None])  # [B,Hkv,n,D]
    dense = np.zeros((B, Hq, Sq, S), F)
    for b in range(B):
        for h in range(Hq):
            for i in range(Sq):
                cols = np.nonzero(match[b, h, i])[0]
                if cols.size == 0:
                    continue
                cosv = r(lane_sum(qunit[b, h, i][None, :] * kn[b, h // G, cols]))
                dense[b, h, i, cols] = collision_prob(cosv, K, L, dtype)
    return match, dense


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
    qcodes, qunit = query_side(q, mean, G, proj, L, K, dtype, meta.get("lsh_query_codes_in"))
    meta["lsh_query_codes"] = qcodes
    match, dense = match_probabilities(qcodes, qunit, state["codes"], k, mean, state["norms"], M, K, L, dtype)
    meta["lsh_match"] = match
    meta["lsh_dense"] = dense
    st.set(mask_ops.merge(st.mask, dense, dtype))


def chunked_step(prm, sink: int, window: int, q, get_chunk, S: int, chunk: int, dtype: str,
                 proj, scaling, on_chunk=None, known_match=None):
    """One decode step of Sink + Local + MagicPig over a sequence too long for the reference's
    own tensors (its packed signatures alone are int64 [B,Hq,S,L], :122-129): the global key
    mean (:175-176) and the global maximum key norm (:352-353) first, then the reference's
    per-key arithmetic chunk by chunk (`key_codes`, `match_probabilities`), the dense mask of
    every chunk merged with the sink / window bands (:593), the attention partial of the chunk,
    and the associative combine of the partials.

    `get_chunk(c0, c1)` returns float32 `(k, v)` [B,Hkv,c1-c0,D].  `on_chunk(c0, c1, mask, codes)`
    (optional) sees every chunk's dense mask [B,Hq,Sq,c1-c0] and key codes.  `known_match(c0, c1)`
    (optional) may return the chunk's matches (bool [B,Hq,Sq,c1-c0]) to spare the chunk the key
    signatures -- by far the largest part of the work -- or None to have them computed; `codes`
    is then None for that chunk.  Returns the output [B,Sq,Hq,D] and the state (mean, M)."""
    from . import attention, mask_ops
    from .sharded import merge_partials

    B, Hq, Sq, D = q.shape
    L, K = prm["lsh_l"], prm["lsh_k"]
    proj = np.asarray(proj, F)
    bounds = [(c0, min(S, c0 + chunk)) for c0 in range(0, S, chunk)]
    mean = None
    if prm.get("center", True):
        total = None
        for c0, c1 in bounds:
            ks_, _ = get_chunk(c0, c1)
            part = np.asarray(ks_, np.float64).sum(axis=2)
            total = part if total is None else total + part
        mean = round_to((total / S).astype(F), dtype)
    Hkv = total.shape[1] if mean is not None else get_chunk(0, 1)[0].shape[1]
    G = Hq // Hkv
    nks, M = [], F(0)
    for c0, c1 in bounds:
        ks_, _ = get_chunk(c0, c1)
        nk = norms(centred(ks_, None if mean is None else mean[:, :, None, :], dtype), dtype)
        nks.append(nk)
        M = F(max(M, nk.max()))
    qcodes, qunit = query_side(q, mean, G, proj, L, K, dtype)
    nums, dens, mxs = [], [], []
    for (c0, c1), nk in zip(bounds, nks):
        ks_, vs_ = get_chunk(c0, c1)
        given = known_match(c0, c1) if known_match is not None else None
        codes = key_codes(ks_, mean, nk, M, proj, L, K, dtype) if given is None else None
        _, dense = match_probabilities(qcodes, qunit, codes, ks_, mean, nk, M, K, L, dtype, match=given)
        cols = np.arange(c0, c1)
        band = np.zeros((B, Hq, Sq, c1 - c0), F)
        band[..., cols < sink] = 1.0
        off = cols[None, :] - np.arange(Sq)[:, None]
        band[..., (off >= S - Sq - window + 1) & (off < S - Sq + 1)] = 1.0
        mask = mask_ops.merge(band, dense, dtype)
        if on_chunk is not None:
            on_chunk(c0, c1, mask, codes)
        num, den, mx = attention.masked_attention(q, ks_, vs_, mask, scaling, dtype, return_partials=True)
        if not mask.any(axis=-1).all():  # a row without any selected key in this chunk
            empty = ~mask.any(axis=-1, keepdims=True)
            num, den, mx = np.where(empty, 0, num), np.where(empty, 0, den), np.where(empty, -np.inf, mx)
        nums.append(num), dens.append(den), mxs.append(mx)
    with np.errstate(invalid="ignore"):
        out = merge_partials(np.stack(nums), np.stack(dens), np.stack(mxs), dtype)
    return out, {"mean": mean, "M": M, "qcodes": qcodes}
