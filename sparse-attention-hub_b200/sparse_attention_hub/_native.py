"""ctypes binding of `libsah_b200.so`, the sm_100a kernel library.

The library is the only compute path of this package: every masker and the
masked-attention step launch its kernels.  There is no fallback; when the
library is missing, or a tensor does not live on a CUDA device, the call
raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import (
    POINTER,
    Structure,
    c_char_p,
    c_float,
    c_int,
    c_int32,
    c_int64,
    c_void_p,
)
from pathlib import Path
from typing import Optional

import torch

SAH_F32 = 0
SAH_BF16 = 1

ACTIVATIONS = {"relu": 0, "silu": 1, "gelu": 2, "tanh": 3}

_PKG_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = Path(os.environ.get("SAH_B200_LIB", _PKG_ROOT / "lib" / "libsah_b200.so"))


class NativeLibraryError(RuntimeError):
    """The sm_100a library is missing, failed to load, or returned an error."""


class AttnSizes(Structure):
    """Mirror of `sah_attn_sizes` (include/sah_b200.h)."""

    _fields_ = [
        ("groups", c_int32),
        ("q_block", c_int32),
        ("rows_per_group", c_int32),
        ("nsplit", c_int32),
        ("ucols_bytes", c_int64),
        ("umemb_bytes", c_int64),
        ("uw_bytes", c_int64),
        ("ucount_bytes", c_int64),
        ("partial_bytes", c_int64),
    ]


_P = c_void_p
_I = c_int
_L = c_int64

# name -> argument types (all functions return int status unless noted)
_SIGNATURES = {
    "sah_mask_fill_band": [_P, _L, _I, _L, _L, _L, _L, _L, _L, _I, _P],
    "sah_mask_fill_bands": [_P, _L, _I, _L, _L, _I, _P, _I, _P],
    "sah_mask_rowscan": [_P, _L, _L, _P, _P, _P],
    "sah_mask_bits_to_indices": [_P, _P, _P, _L, _L, _L, _P, _P],
    "sah_mask_bits_to_dense": [_P, _P, _P, _P, _I, _L, _L, _L, _P, _P],
    "sah_mask_dense_to_bits": [_P, _I, _L, _L, _L, _P, _P],
    "sah_mask_dense_gather_data": [_P, _I, _P, _P, _P, _L, _L, _L, _P, _P],
    "sah_mask_or": [_P, _P, _L, _P, _P],
    "sah_mask_sample_data": [_P, _P, _P, _P, _P, _P, _I, _L, _L, _L, _P, _P],
    "sah_mask_scatter_samples": [_P, _P, _L, _L, _L, _L, _P, _P],
    "sah_hash_encode": [_P, _I, _L, _L, _L, _I, _I, _I, _L, _L, _L, _I, POINTER(c_int),
                        POINTER(c_void_p), POINTER(c_void_p), _I, _P, _P, _P],
    "sah_hash_topk": [_P, _L, _P, _I, _P, _I, _L, _L, _L, _I, _I, _I, _L, _L, _P, _L, _P, _P],
    "sah_qk_scores": [_P, _P, _I, _L, _L, _L, _L, _L, _L, _I, _I, _I, _I, _L, _I, _P, _L, _L,
                      _L, _P, _P],
    "sah_topk_select": [_P, _I, _L, _L, _L, _L, _L, _P, _L, _P, _P],
    "sah_topk_select_ws_bytes": [_L, _L],  # returns int64
    "sah_topk_sel_hist_offset": [_L, _L],  # returns int64
    "sah_topk_sel_begin": [_L, _L, _L, _P, _L, _P],
    "sah_topk_sel_hist": [_P, _I, _L, _L, _L, _L, _L, _P, _P, _I, _P],
    "sah_topk_sel_pick": [_L, _L, _P, _I, _I, _P, _P],
    "sah_topk_sel_emit": [_P, _I, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P],
    "sah_topk_select_ws": [_P, _I, _L, _L, _L, _L, _L, _P, _L, _P, _P, _L, _P],
    "sah_attn_query_sizes": [_I, _I, _I, _I, _L, _I, _I, _I, POINTER(AttnSizes)],
    "sah_attn_plan": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _L, POINTER(AttnSizes), _P, _P,
                      _P, _P, _P],
    "sah_masked_attention": [_P, _P, _P, _I, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _I, _I, _I,
                             _L, _I, c_float, _P, _L, _L, _L, _P, POINTER(AttnSizes), _P, _P, _P,
                             _P, _P, _P, _P, _P],
    "sah_attn_merge_parts": [_P, _I, _I, _I, _I, _I, _P, _I, _P, _P],
    "sah_attn_plan_lsh": [_P, _P, _P, _L, _P, _I, _I, _I, _I, _L, _L, POINTER(AttnSizes), _P, _P, _P,
                          _P, _P],
    "sah_masked_attention_lsh": [_P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _I, _I, _I, _L,
                                 _I, c_float, _P, _L, _L, _L, _P, POINTER(AttnSizes), _P, _P, _P, _P,
                                 _P, _P, _P, _P, _P, _P, _P, _P],
    "sah_mask_unit_data": [_P, _P, _P, _P, _I, _L, _L, _P, _P],
    "sah_mask_rowwise_scatter": [_P, _P, _I, _L, _L, _L, _P, _P, _P],
    "sah_mask_flat_add": [_P, _P, _I, _L, _L, _P, _P],
    "sah_mask_clamp_to_dense": [_P, _I, _L, _P, _P],
    "sah_attn_select_kernel": [_I],
    "sah_wait_selftest": [_I, _P, _P, _P],
    "sah_attn_exchange_bytes": [_I, _I, _I, _I, _I],  # returns int64
    "sah_attn_exchange_merge": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _P, _P],
    "sah_attn_gather_probe": [_P, _P, _L, _L, _L, _L, _L, _L, _I, _I, _I, _L, _I, POINTER(AttnSizes),
                              _P, _P, _P, _P],
    "sah_adaptive_budget": [_P, _I, c_float, _P, _L, _L, _L, _P, _P, _P, _P, _I, _I, _I, _L, _L, _L,
                            _L, _L, ctypes.c_uint64, _P, _P, c_float, c_float, _P, _P, _P, _P],
    "sah_topp_select": [_P, _I, c_float, _P, _L, _L, _L, _I, _I, _I, _L, _L, _P, c_float, _P, _I, _P, _P],
    "sah_quest_page_minmax": [_P, _I, _L, _L, _L, _I, _I, _L, _I, _I, _L, _L, _P, _P, _P],
    "sah_quest_scores": [_P, _I, _L, _L, _L, _P, _P, _L, _I, _I, _I, _I, _L, _I, _I, _P, _L, _L, _L, _P, _P],
    "sah_quest_expand": [_P, _L, _P, _P, _I, _L, _L, _L, _I, _I, _I, _L, _L, _I, _P, _P],
    "sah_sample_scatter": [_P, _L, _P, ctypes.c_uint64, _L, _L, _L, _L, _I, _P, _P],
    "sah_hash_hist": [_P, _L, _P, _I, _I, _I, _I, _L, _L, _I, _P, _P, _P, _P],
    "sah_hash_scores_bytes": [_L, _L],  # returns int64
    "sah_hash_shard_plan": [_P, _I, _I, _I, _L, _L, _P, _P, _P],
    "sah_hash_emit": [_P, _L, _P, _I, _I, _I, _I, _L, _L, _I, _P, _P, _P, _P, _P, _P],
    "sah_hash_topk_ws_bytes": [_L, _L, _I],  # returns int64
    "sah_hash_topk_ws": [_P, _L, _P, _I, _I, _I, _I, _L, _L, _P, _L, _P, _P, _L, _I, _P],
    "sah_mask_merge_bits": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _L, _P, _P],
    "sah_mask_merge_data": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _L, _L, _P, _P, _P, _P, _P],
    "sah_lsh_key_sums": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _I, _P, _P],
    "sah_lsh_key_stats": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _I, _P, _L, _P, _P, _I, _P],
    "sah_lsh_key_sign_tc_ws_bytes": [_I, _I, _L],  # returns int64
    "sah_lsh_key_sign_tc": [_P, _L, _L, _L, _I, _I, _L, _L, _I, _P, _P, _P, _P, _I, _I, _L, _P, _P, _L, _I, _P],
    "sah_lsh_key_sign": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _I, _P, _P, _P, _P, _I, _I, _L, _P, _P],
    "sah_lsh_query": [_P, _I, _L, _L, _L, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _P, _P, _P, _P],
    "sah_lsh_match": [_P, _L, _P, _I, _I, _I, _I, _I, _I, _L, _L, _P, _P, _P],
    "sah_lsh_key_den": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _I, _P, _P, _L, _P, _P, _P, _I, _P],
    "sah_lsh_prob": [_P, _I, _L, _L, _L, _I, _I, _I, _I, _I, _P, _P, _P, _L, _P, _P, _P, _P, _P, _L,
                     _I, _I, _P, _P, _I, _P],
    "sah_pq_assign_tc": [_P, _L, _L, _L, _I, _I, _L, _L, _L, _I, _I, _I, _P, _P, _L, _P, _I, _P],
    "sah_pq_assign": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _L, _I, _I, _I, _P, _P, _L, _I, _P],
    "sah_pq_accumulate": [_P, _I, _L, _L, _L, _I, _I, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P],
    "sah_pq_update": [_P, _I, _L, _L, _L, _I, _I, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P],
    "sah_pq_scores_ws_bytes": [_I, _I, _I, _I, _I, _I],  # returns int64
    "sah_pq_scores": [_P, _I, _L, _L, _L, _P, _P, _L, _I, _I, _I, _I, _L, _L, _L, _I, _I, _I, _P,
                      _P, _L, _P],
    "sah_masked_attention_static": [_P, _P, _P, _P, _I, _L, _L, _L, _L, _L, _L, _L, _L, _L, _I, _I,
                                    _I, _I, _L, _L, _I, c_float, _P, _L, _L, _L, _P, _I, _P, _P],
    "sah_profile_enable": [_I],
    "sah_profile_read": [_I, POINTER(c_float), POINTER(c_int)],
}

PROFILE_SLOTS = {"attention": 0, "hash_topk": 1, "hash_encode": 2, "qk_scores": 3,
                 "topk_select": 4, "attn_plan": 5, "attn_merge": 6, "other": 7, "lsh_match": 8, "lsh_prob": 9,
                 "pq_scores": 10, "adaptive_budget": 11, "topp_select": 12, "quest_scores": 13}

EXPORTED_SYMBOLS = sorted(list(_SIGNATURES) + ["sah_version", "sah_last_error", "sah_launch_count",
                                                 "sah_attn_last_kernel"])

_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load the shared library once; raise NativeLibraryError when it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise NativeLibraryError(
            f"{LIB_PATH} not found: build it with "
            f"`python {_PKG_ROOT / 'build.py'}` (needs nvcc; no GPU required to build)"
        )
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError as exc:  # pragma: no cover - depends on the host
        raise NativeLibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.sah_topk_select_ws_bytes.restype = c_int64
    lib.sah_attn_exchange_bytes.restype = c_int64
    lib.sah_lsh_key_sign_tc_ws_bytes.restype = c_int64
    lib.sah_pq_scores_ws_bytes.restype = c_int64
    lib.sah_topk_sel_hist_offset.restype = c_int64
    lib.sah_hash_topk_ws_bytes.restype = c_int64
    lib.sah_hash_scores_bytes.restype = c_int64
    lib.sah_version.restype = c_char_p
    lib.sah_last_error.restype = c_char_p
    lib.sah_attn_last_kernel.restype = c_char_p
    lib.sah_attn_last_kernel.argtypes = []
    lib.sah_launch_count.restype = ctypes.c_longlong
    lib.sah_launch_count.argtypes = []
    _lib = lib
    return lib


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(load().sah_launch_count())


def profile_enable(on: bool) -> None:
    check(load().sah_profile_enable(int(on)), "sah_profile_enable")


def profile_read(slot: str):
    """(total milliseconds, launches) recorded for a kernel slot since the last read."""
    ms, n = c_float(0.0), c_int(0)
    check(load().sah_profile_read(PROFILE_SLOTS[slot], ctypes.byref(ms), ctypes.byref(n)),
          "sah_profile_read")
    return float(ms.value), int(n.value)


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().sah_last_error().decode("utf-8", "replace")
        kind = {1: "invalid argument", 2: "unsupported", 3: "CUDA error", 4: "workspace"}.get(
            status, f"status {status}"
        )
        if status == 2:
            raise NotImplementedError(f"{what}: {msg}")
        raise NativeLibraryError(f"{what}: {kind}: {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return SAH_F32
    if dtype == torch.bfloat16:
        return SAH_BF16
    raise NotImplementedError(
        f"the sm_100a kernels compute in float32 or bfloat16, got {dtype}"
    )


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise NativeLibraryError(
            f"{name} lives on {t.device}; the native path runs on CUDA devices only "
            "and has no CPU fallback"
        )


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_of(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_sm_count_cache: dict = {}


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count_cache:
        _sm_count_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count_cache[idx]
