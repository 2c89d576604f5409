"""bfloat16 arithmetic emulated on float32 arrays (round-to-nearest-even)."""

import numpy as np


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 array -> nearest bfloat16 value, returned as float32."""
    f = np.ascontiguousarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    out = r.astype(np.uint32).view(np.float32).reshape(f.shape)
    nan = np.isnan(f)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out


def bits_of(x: np.ndarray) -> np.ndarray:
    """bf16-valued float32 array -> uint16 bit patterns."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def from_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round to the value grid of `dtype` ("bf16" or "f32")."""
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(dtype)


def finfo_min(dtype: str) -> np.float32:
    """torch.finfo(dtype).min as float32."""
    if dtype == "bf16":
        return np.float32(-3.3895313892515355e38)
    return np.finfo(np.float32).min
