"""Sampling maskers restated (research_attention/maskers/sampling/implementations/
adaptive_sampling.py, random_sampling.py; utils/mask_attention_utils.py:105-184)."""

import numpy as np

from . import mask_ops
from .bf16 import bits_of, from_bits, round_bf16, round_to

_EXP_TABLE = None


def exp_table() -> np.ndarray:
    """uint16[65536]: bf16 bits of x -> bf16 bits of exp(x) (float64, rounded through float32)."""
    global _EXP_TABLE
    if _EXP_TABLE is None:
        with np.errstate(invalid="ignore"):
            x = from_bits(np.arange(65536, dtype=np.uint32).astype(np.uint16)).astype(np.float64)
        with np.errstate(over="ignore", invalid="ignore"):
            y = np.where(np.isnan(x), x, np.exp(x))
            t = bits_of(round_bf16(y.astype(np.float32)))
        t[np.isnan(y)] = 0x7FC0
        _EXP_TABLE = t
    return _EXP_TABLE


def exp_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return from_bits(exp_table()[bits_of(x)])
    # fp32: double-precision exp rounded once (the kernels do the same)
    return np.exp(np.asarray(x, np.float32).astype(np.float64)).astype(np.float32)


# ---- Philox4x32-10, first output word --------------------------------------------------
def philox_u32(seed: int, index: np.ndarray) -> np.ndarray:
    idx = np.asarray(index, np.uint64)
    c0 = (idx & 0xFFFFFFFF).astype(np.uint64)
    c1 = (idx >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0 = np.uint64(seed & 0xFFFFFFFF)
    k1 = np.uint64((seed >> 32) & 0xFFFFFFFF)
    M0, M1, MASK = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & MASK
        k1 = (k1 + np.uint64(0xBB67AE85)) & MASK
    return c0.astype(np.uint32)


def draw_columns(seed: int, index: np.ndarray, start: int, n: int) -> np.ndarray:
    """start + floor(u * n / 2^32)."""
    u = philox_u32(seed, index).astype(np.uint64)
    return (start + ((u * np.uint64(n)) >> np.uint64(32))).astype(np.int64)


# ---- fixed-order sum -------------------------------------------------------------------
def fixed_sum(x: np.ndarray) -> np.float32:
    """Sum of a 1-D float32 array in the order the kernels use: element j goes to partial
    j mod 1024 (ascending j), then xor trees (16, 8, 4, 2, 1) over the 32 lanes of each warp
    and over the 32 warp sums."""
    x = np.asarray(x, np.float32)
    pad = (-x.size) % 1024
    if pad:
        x = np.concatenate([x, np.zeros(pad, np.float32)])
    p = np.zeros(1024, np.float32)
    for chunk in x.reshape(-1, 1024):
        p = p + chunk
    p = p.reshape(32, 32)
    lanes = np.arange(32)
    for off in (16, 8, 4, 2, 1):
        p = p + p[:, lanes ^ off]
    w = p[:, 0].copy()
    for off in (16, 8, 4, 2, 1):
        w = w + w[lanes ^ off]
    return np.float32(w[0])


# ---- adaptive sampling -----------------------------------------------------------------
def sampling_range(S: int, init_offset, local_offset):
    start = int(init_offset * S) if isinstance(init_offset, float) else init_offset
    end = S - (int(local_offset * S) if isinstance(local_offset, float) else local_offset)
    return start, end, end - start


def base_count(rate, n: int) -> int:
    return max(2, rate) if isinstance(rate, int) else max(2, int(rate * n))


def adaptive_budget_row(scores_row, scaling, bias_row, prev_row, start, end, nb, base_cols,
                        delta_ppf, epsilon, dtype):
    """One row of AdaptiveSamplingMasker.add_mask (:304-407) up to the budget.
    scores_row: unscaled q.k in dtype; prev_row: dense previous mask row or None (empty/full)."""
    r = lambda x: round_to(np.asarray(x, np.float32), dtype)  # noqa: E731
    rs = lambda x: np.float32(round_to(np.array([x], np.float32), dtype)[0])  # noqa: E731
    f32 = np.float32
    n = end - start
    t = r(np.asarray(scores_row, np.float32) * f32(scaling))
    if bias_row is not None:
        t = r(t + np.asarray(bias_row, np.float32)[: t.size])
    mx = t.max()
    e = exp_dtype(r(t - mx), dtype)
    if prev_row is None:
        static_den = rs(fixed_sum(e))
    else:
        w = mask_ops.inv_weights(prev_row, dtype)
        static_den = rs(fixed_sum(np.where(prev_row != 0, r(e * w), f32(0))))
    vals = e[np.asarray(base_cols)]
    mean = f32(fixed_sum(vals) / f32(nb))
    dev = (vals - mean).astype(np.float32)
    var = f32(fixed_sum(dev * dev) / f32(nb - 1))
    sd = max(rs(np.sqrt(var)), rs(1e-8))
    p_base = rs(nb / n)
    w_base = f32(mask_ops.inv_weights(np.array([p_base], np.float32), dtype)[0])
    member = np.zeros(e.size, bool)
    member[np.asarray(base_cols)] = True
    sampled_den = rs(fixed_sum(np.where(member, r(e * w_base), f32(0))))
    est = rs(static_den + sampled_den)
    err = max(rs(f32(epsilon) * est), rs(1e-8))
    num = rs(rs(f32(delta_ppf) * sd) * f32(n))
    ratio = rs(num / err)
    b2 = rs(ratio * ratio)
    clamped = min(max(b2, f32(1.0)), rs(n))
    budget = int(min(max(int(clamped), nb), n))
    prob = rs(f32(budget) / f32(n))
    return budget, prob, (static_den, sd, est, b2)
