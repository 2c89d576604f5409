"""Dense-mask arithmetic of the reference's Mask (sparse_attention/utils/mask.py)."""

import numpy as np

from .bf16 import round_to


def effective_size(size, seq_len_keys: int) -> int:
    """ResearchMasker._calculate_effective_size (maskers/base.py:152-158)."""
    return int(size * seq_len_keys) if isinstance(size, float) else int(size)


def sink(mask: np.ndarray, sink_size: int) -> np.ndarray:
    """SinkMasker.get_updated_mask_dense (fixed/implementations/basic_fixed.py:354-363)."""
    out = mask.copy()
    out[..., :sink_size] = 1.0
    return out


def local(mask: np.ndarray, window: int) -> np.ndarray:
    """LocalMasker.update_core (basic_fixed.py:48-67): band set to 1, future positions to 0."""
    Sq, S = mask.shape[-2], mask.shape[-1]
    off = np.arange(S)[None, :] - np.arange(Sq)[:, None]
    lo, hi = S - Sq - window + 1, S - Sq + 1
    out = mask.copy()
    out[..., (off >= lo) & (off < hi)] = 1.0
    out[..., off >= hi] = 0.0
    return out


def merge(a: np.ndarray, b: np.ndarray, dtype: str) -> np.ndarray:
    """Mask.merge_mask_dense (utils/mask.py:875-877): clamp(a + b, 0, 1) in the mask dtype."""
    return np.clip(round_to(a + b, dtype), 0.0, 1.0).astype(np.float32)


def inv_weights(mask: np.ndarray, dtype: str) -> np.ndarray:
    """Mask.apply_inv_mask_dense factor (utils/mask.py:737-739):
    1 / (m + 1e-6) * (m != 0), each op rounded to the mask dtype."""
    m = np.asarray(mask, dtype=np.float32)
    s = round_to(m + np.float32(1e-6), dtype)
    with np.errstate(divide="ignore"):
        w = round_to(np.float32(1.0) / s, dtype)
    return np.where(m != 0, w, np.float32(0.0)).astype(np.float32)


def to_csr(mask: np.ndarray):
    """Mask.get_index_mask for a dense mask (utils/mask.py:553-573):
    flat ascending int64 indices, ptr (rows+1), data."""
    S = mask.shape[-1]
    flat = mask.reshape(-1)
    idx = np.flatnonzero(flat).astype(np.int64)
    counts = np.count_nonzero(mask.reshape(-1, S), axis=1)
    ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    return idx, ptr, flat[idx].astype(np.float32)


def from_row_wise_idx(shape, row_idx: np.ndarray, row_vals: np.ndarray) -> np.ndarray:
    """Mask.create_from_row_wise_idx, dense mode (utils/mask.py:335-395): each row's values are
    scattered to its columns; of several entries naming one column the last one stays."""
    S = shape[-1]
    idx = np.asarray(row_idx).reshape(-1, row_idx.shape[-1])
    vals = np.asarray(row_vals, dtype=np.float32).reshape(idx.shape)
    out = np.zeros((idx.shape[0], S), dtype=np.float32)
    for r in range(idx.shape[0]):
        for j in range(idx.shape[1]):
            out[r, idx[r, j]] = vals[r, j]
    return out.reshape(shape)


def merge_sparse(a: np.ndarray, b: np.ndarray, dtype: str):
    """Mask.merge_mask_sparse (utils/mask.py:893-1062) for two index-form masks given densely:
    the entries of both are concatenated, sorted by flat index, duplicates summed in the mask
    dtype and clamped to [0, 1]; every index either operand stored stays stored.  Returns the
    CSR triple of the result."""
    S = a.shape[-1]
    fa, fb = a.reshape(-1), b.reshape(-1)
    stored = (fa != 0) | (fb != 0)
    idx = np.flatnonzero(stored).astype(np.int64)
    data = np.clip(round_to(fa[idx] + fb[idx], dtype), 0.0, 1.0).astype(np.float32)
    counts = stored.reshape(-1, S).sum(axis=1)
    ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    return idx, ptr, data
