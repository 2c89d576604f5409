"""Masked attention over a `Mask`.

`get_masked_attention_output` is the hot entry point
(reference: sparse_attention_hub/sparse_attention/utils/mask_attention_utils.py:406-491).
It launches the sm_100a plan + gather-attention kernels: only the K/V rows the
mask selects are read, every row once per KV group, softmax in fp32 with the
inverse mask weights of `Mask.apply_inv_mask` in the denominator and the
numerator.  The row maximum the reference takes over all keys cancels between
numerator and denominator, so the kernel's running maximum over the selected
keys yields the same output.

The remaining functions of the reference module (`apply_inv_mask_sum`,
`create_sampling_mask_with_per_head_budget`, numerator / denominator helpers,
`get_true_attention_output`) are kept for user code that imports them; they are
plain tensor expressions on whatever device their arguments live on and the
native path does not call them.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Any, Dict, Optional, Tuple, Union

import torch
from torch import nn

from ... import _native
from .kv_utils import _get_num_key_value_groups, repeat_kv
from .mask import Mask, NativeBits, words_per_row

_workspace_cache: Dict[Tuple, Dict[str, torch.Tensor]] = {}


def _bias_args(attention_mask: Optional[torch.Tensor], dtype: torch.dtype, n_keys: int):
    """(tensor kept alive, pointer, stride_b, stride_h, stride_q) of the additive bias."""
    if attention_mask is None:
        return None, None, 0, 0, 0
    am = attention_mask
    if am.dim() != 4:
        raise ValueError(f"attention_mask must be 4-D [B, 1 or H, Sq, Sk], got {tuple(am.shape)}")
    if am.shape[-1] < n_keys:
        raise ValueError(f"attention_mask covers {am.shape[-1]} keys, need {n_keys}")
    if am.dtype != dtype:
        am = am.to(dtype)
    if am.stride(-1) != 1:
        am = am.contiguous()
    sb = am.stride(0) if am.shape[0] > 1 else 0
    sh = am.stride(1) if am.shape[1] > 1 else 0
    sq = am.stride(2) if am.shape[2] > 1 else 0
    return am, am.data_ptr(), sb, sh, sq


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _workspace(device: torch.device, sizes: _native.AttnSizes, key: Tuple) -> Dict[str, torch.Tensor]:
    ws = _workspace_cache.get(key)
    if ws is None:
        if len(_workspace_cache) > 16:
            _workspace_cache.clear()
        ws = {
            "ucols": torch.empty(max(1, sizes.ucols_bytes // 4), dtype=torch.int32, device=device),
            "umemb": torch.empty(max(1, sizes.umemb_bytes // 2), dtype=torch.int16, device=device),
            "uw": (torch.empty(sizes.uw_bytes // 4, dtype=torch.float32, device=device)
                   if sizes.uw_bytes > 0 else None),
            # zero-filled once: it ends with the merge tickets, which the kernel keeps at zero
            "ucount": torch.zeros(max(1, sizes.ucount_bytes // 4), dtype=torch.int32, device=device),
            "partial": torch.empty(max(1, sizes.partial_bytes // 4), dtype=torch.float32,
                                   device=device),
        }
        _workspace_cache[key] = ws
    return ws


def native_masked_attention(
    queries: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    sinks: Optional[torch.Tensor],
    scaling: float,
    sparse_attention_mask: Mask,
    return_partials: bool = False,
):
    """Run plan + gather attention; returns `out [B, Sq, Hq, D]` in the query dtype.

    With `return_partials=True` also returns a float32 `[rows, D + 2]` tensor: per mask row
    the unnormalised accumulator, the running maximum and the denominator, which is what a
    sequence-sharded caller all-gathers (one buffer, one collective) and merges.
    """
    _native.require_cuda(queries, "queries")
    _native.require_cuda(keys, "keys")
    _native.require_cuda(values, "values")
    lib = _native.load()
    B, Hq, Sq, D = queries.shape
    Hkv, S = keys.shape[1], keys.shape[2]
    if values.shape[2] != S or values.shape[1] != Hkv:
        raise ValueError("keys and values disagree on heads or length")
    _get_num_key_value_groups(queries, keys)
    dtype = queries.dtype
    code = _native.dtype_code(dtype)
    if keys.dtype != dtype or values.dtype != dtype:
        raise ValueError("queries, keys and values must share one dtype")
    dev = queries.device
    st = _native.stream_of(dev)

    q, k, v = _rowmajor(queries), _rowmajor(keys), _rowmajor(values)
    mask = sparse_attention_mask
    if tuple(mask.shape) != (B, Hq, Sq, S):
        raise ValueError(f"mask shape {mask.shape} does not match attention shape {(B, Hq, Sq, S)}")
    if mask.is_full or mask.is_empty:
        # both mean "no masking" to the attention step (utils/mask.py:733-735)
        nb = Mask.create_full_mask(mask.shape, dtype, dev).native_bits()
    else:
        nb = mask.native_bits()
    # a MagicPig mask may come with what the kernel needs to evaluate its weights in place
    payload = nb.deferred
    has_data = 2 if payload is not None else int(nb.data is not None)
    if has_data == 1:
        nb.ensure_scan()

    sizes = _native.AttnSizes()
    _native.check(lib.sah_attn_query_sizes(B, Hq, Hkv, Sq, S, D, has_data,
                                           _native.sm_count(dev), ctypes.byref(sizes)),
                  "sah_attn_query_sizes")
    if payload is not None and (sizes.rows_per_group > 4 or dtype != torch.bfloat16):
        payload, has_data = None, int(nb.data is not None)  # materialises the weights
        nb.ensure_scan()
        _native.check(lib.sah_attn_query_sizes(B, Hq, Hkv, Sq, S, D, has_data,
                                               _native.sm_count(dev), ctypes.byref(sizes)),
                      "sah_attn_query_sizes")
    # scratch is reused across calls of one shape; calls that could overlap on the device
    # (another stream, another host thread) get their own
    key = (dev.index, st, threading.get_ident(), B, Hq, Hkv, Sq, S, D, has_data)
    ws = _workspace(dev, sizes, key)
    if "groups" not in ws:  # where the kernel's error word sits behind the counters and tickets
        nchunks = (words_per_row(S) + 31) // 32
        ws["groups"], ws["err_index"] = sizes.groups, 2 * sizes.groups + sizes.groups * nchunks
    keep, bias_ptr, bsb, bsh, bsq = _bias_args(attention_mask, dtype, S)
    sink_t = None
    if sinks is not None:
        if sinks.dim() != 1 or sinks.shape[0] != Hq:
            raise ValueError(f"sinks must be 1D tensor of shape [H], got {tuple(sinks.shape)}")
        sink_t = sinks.to(device=dev, dtype=torch.float32).contiguous()
    out = torch.empty((B, Sq, Hq, D), dtype=dtype, device=dev)
    rows = B * Hq * Sq
    part = torch.empty((rows, D + 2), dtype=torch.float32, device=dev) if return_partials else None
    strides = (q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
               v.stride(0), v.stride(1), v.stride(2))
    try:
        if payload is not None:
            sig = payload.sig
            _native.check(
                lib.sah_attn_plan_lsh(payload.match_bits.data_ptr(), _native.ptr(payload.unit_bits),
                                      sig.dens.data_ptr(), sig.capacity, sig.max_norm.data_ptr(), B, Hq,
                                      Hkv, Sq, S, payload.match_bits.shape[-1], ctypes.byref(sizes),
                                      ws["ucols"].data_ptr(), ws["umemb"].data_ptr(),
                                      ws["uw"].data_ptr(), ws["ucount"].data_ptr(), st),
                "sah_attn_plan_lsh")
            dump = _weight_dump.get("request")
            if dump is not None:
                dump = torch.zeros(sizes.groups * S * sizes.rows_per_group, dtype=torch.float32, device=dev)
                _weight_dump["weights"] = dump
            _native.check(
                lib.sah_masked_attention_lsh(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), *strides, B, Hq, Hkv, Sq, S, D,
                    float(scaling), bias_ptr, bsb, bsh, bsq, _native.ptr(sink_t), ctypes.byref(sizes),
                    ws["ucols"].data_ptr(), ws["umemb"].data_ptr(), ws["uw"].data_ptr(),
                    ws["ucount"].data_ptr(), ws["partial"].data_ptr(), payload.qhat.data_ptr(),
                    payload.qmu.data_ptr(), payload.weight_table.data_ptr(), out.data_ptr(),
                    _native.ptr(part), _native.ptr(dump), st),
                "sah_masked_attention_lsh")
        else:
            _native.check(
                lib.sah_attn_plan(nb.bits.data_ptr(), _native.ptr(nb.data), _native.ptr(nb.wpre),
                                  _native.ptr(nb.ptr), code, B, Hq, Hkv, Sq, S, nb.words,
                                  ctypes.byref(sizes), ws["ucols"].data_ptr(), ws["umemb"].data_ptr(),
                                  _native.ptr(ws["uw"]) if has_data else None, ws["ucount"].data_ptr(), st),
                "sah_attn_plan")
            _native.check(
                lib.sah_masked_attention(
                    q.data_ptr(), k.data_ptr(), v.data_ptr(), code, *strides,
                    B, Hq, Hkv, Sq, S, D, float(scaling), bias_ptr, bsb, bsh, bsq,
                    _native.ptr(sink_t), ctypes.byref(sizes), ws["ucols"].data_ptr(),
                    ws["umemb"].data_ptr(), _native.ptr(ws["uw"]) if has_data else None,
                    ws["ucount"].data_ptr(), ws["partial"].data_ptr(), out.data_ptr(),
                    _native.ptr(part), st),
                "sah_masked_attention")
    except Exception:
        # a refused launch may leave the merge tickets of this scratch non-zero
        _workspace_cache.pop(key, None)
        raise
    del keep
    _last_plan["ucount"] = ws["ucount"][: sizes.groups]
    _last_plan["ws"] = ws
    _last_plan["sizes"] = (sizes.groups, sizes.rows_per_group, S)
    _last_plan["attn_sizes"] = sizes
    if return_partials:
        return out, part
    return out


# Test hook: set _weight_dump["request"] to anything but None and the next attention call over a
# MagicPig mask with in-kernel weights leaves the weights it used in _weight_dump["weights"]
# (float32 [groups * S * rows_per_group], union-list order; see last_union_list()).
_weight_dump: Dict[str, Any] = {"request": None, "weights": None}

_last_plan: Dict[str, Any] = {"ucount": None, "ws": None, "sizes": None}


def last_union_counts() -> Optional[torch.Tensor]:
    """int32 [groups]: distinct K/V rows the most recent attention call gathered per KV group
    (valid once the launching stream has run; used for bandwidth accounting)."""
    return _last_plan["ucount"]


def attention_wait_errors() -> int:
    """How many cached attention workspaces carry a set error word (a bounded wait of the
    tensor-map copy stage ran out in some launch that used them); reads device memory."""
    n = 0
    for ws in _workspace_cache.values():
        groups = ws.get("groups")
        if groups is not None:
            n += int(ws["ucount"][ws["err_index"]].item() != 0)
    return n


def last_union_list():
    """(ucols int32 [groups, S], umemb int16 [groups, S], ucount int32 [groups], rows per group)
    of the most recent attention call: the ascending union of the columns each KV group
    gathered, and which of the group's rows selected each."""
    ws, (groups, R, S) = _last_plan["ws"], _last_plan["sizes"]
    return (ws["ucols"][: groups * S].view(groups, S), ws["umemb"][: groups * S].view(groups, S),
            ws["ucount"][:groups], R)


ATTENTION_KERNELS = {"auto": -1, "mma": 0, "umma": 1}


def select_attention_kernel(which: str) -> str:
    """Choose the bfloat16 attention kernel of this process (`sah_attn_select_kernel`): "mma"
    (per-warp mma.sync over 16-key tiles), "umma" (tcgen05 over 128-key tiles, head dim 128) or
    "auto" (the library decides per call).  Returns the previous choice."""
    if which not in ATTENTION_KERNELS:
        raise ValueError(f"attention kernel {which!r}: one of {sorted(ATTENTION_KERNELS)}")
    prev = _native.load().sah_attn_select_kernel(ATTENTION_KERNELS[which])
    return {v: k for k, v in ATTENTION_KERNELS.items()}[prev]


def last_attention_kernel() -> str:
    """Name of the kernel that the most recent attention call of this process launched."""
    return _native.load().sah_attn_last_kernel().decode()


def gather_probe(keys: torch.Tensor, values: torch.Tensor, seq_len_queries: int = 1) -> None:
    """Launch the row-gather probe (`sah_attn_gather_probe`) on the union list of the most recent
    bfloat16 attention call over these keys and values: the copy pipeline of the attention kernel
    without its arithmetic.  Timed by the caller (profile slot "other"), it gives the ceiling
    that the gather of exactly those rows allows."""
    lib = _native.load()
    ws, sizes = _last_plan["ws"], _last_plan["attn_sizes"]
    k, v = _rowmajor(keys), _rowmajor(values)
    B, Hkv, S, D = k.shape
    sink = ws.setdefault("probe_sink", torch.zeros(1, dtype=torch.int32, device=k.device))
    _native.check(
        lib.sah_attn_gather_probe(k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2),
                                  v.stride(0), v.stride(1), v.stride(2), B, Hkv, seq_len_queries, S, D,
                                  ctypes.byref(sizes), ws["ucols"].data_ptr(), ws["ucount"].data_ptr(),
                                  sink.data_ptr(), _native.stream_of(k.device)),
        "sah_attn_gather_probe")


def merge_attention_partials(parts: torch.Tensor, batch: int, heads: int, seq_len_queries: int,
                             dtype: torch.dtype, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Combine `[n_parts, rows, D + 2]` partials (accumulator, max, denominator per row) of
    `native_masked_attention(..., return_partials=True)` over disjoint key ranges."""
    _native.require_cuda(parts, "parts")
    lib = _native.load()
    n_parts, rows, ld = parts.shape
    D = ld - 2
    dev = parts.device
    out = torch.empty((batch, seq_len_queries, heads, D), dtype=dtype, device=dev)
    sink_t = None if sinks is None else sinks.to(device=dev, dtype=torch.float32).contiguous()
    # named, so that a copy outlives the launch (a temporary would be freed, and its memory
    # handed to the next allocation, as soon as its address had been read)
    parts_c = parts.contiguous()
    _native.check(
        lib.sah_attn_merge_parts(parts_c.data_ptr(), n_parts, batch, heads, seq_len_queries, D,
                                 _native.ptr(sink_t), _native.dtype_code(dtype), out.data_ptr(),
                                 _native.stream_of(dev)),
        "sah_attn_merge_parts")
    return out


def get_masked_attention_output(
    module: Optional[nn.Module],
    queries: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    sinks: Optional[torch.Tensor],
    scaling: float,
    dropout: float,
    sparse_attention_mask: Mask,
    return_attention_weights: bool = False,
    **kwargs: Dict[str, Any],
) -> Union[torch.Tensor, Tuple[torch.Tensor, Optional[torch.Tensor]]]:
    """Weighted-softmax attention over the mask; output `[B, Sq, Hq, D]` in the query dtype.

    With `return_attention_weights=True` the second element is the dense
    probability tensor `[B, Hq, Sq, Sk]`, produced from the mask's dense form
    (an O(Sk) write the decode path avoids by not asking for it).
    """
    training = module.training if module is not None else False
    if dropout > 0.0 and training:
        raise NotImplementedError("attention dropout is a training feature; the native path is inference-only")
    out = native_masked_attention(queries, keys, values, attention_mask, sinks, scaling,
                                  sparse_attention_mask)
    if not return_attention_weights:
        return out
    weights = _dense_attention_probabilities(queries, keys, attention_mask, sinks, scaling,
                                             sparse_attention_mask)
    return out, weights


# ---------------------------------------------------------------------------
# Interop helpers (tensor expressions; not on the native path)
# ---------------------------------------------------------------------------
def _compute_masked_exp_attention_weights(
    queries: torch.Tensor,
    keys: torch.Tensor,
    attention_mask: Optional[torch.Tensor],
    scaling: float,
    sparse_attention_mask: Mask,
    dropout: float = 0.0,
    training: bool = False,
) -> torch.Tensor:
    """exp(logits - rowmax) with inverse mask weights applied, `[B, Hq, Sq, Sk]` fp32."""
    k = repeat_kv(keys, _get_num_key_value_groups(queries, keys)).to(torch.float32)
    logits = torch.matmul(queries.to(torch.float32), k.transpose(2, 3)) * scaling
    if attention_mask is not None:
        logits = logits + attention_mask[:, :, :, : k.shape[-2]].to(torch.float32)
    logits = logits - logits.max(dim=-1, keepdim=True)[0]
    weights = sparse_attention_mask.apply_inv_mask(torch.exp(logits))
    if dropout > 0.0 and training:
        weights = torch.nn.functional.dropout(weights, p=dropout, training=training)
    return weights


def _dense_attention_probabilities(queries, keys, attention_mask, sinks, scaling, mask: Mask):
    w = _compute_masked_exp_attention_weights(queries, keys, attention_mask, scaling, mask)
    den = w.sum(dim=-1, keepdim=True)
    if sinks is not None:
        k = repeat_kv(keys, _get_num_key_value_groups(queries, keys)).to(torch.float32)
        logits = torch.matmul(queries.to(torch.float32), k.transpose(2, 3)) * float(scaling)
        if attention_mask is not None:
            logits = logits + attention_mask[:, :, :, : k.shape[-2]].to(torch.float32)
        old_max = logits.max(dim=-1, keepdim=True).values
        s = sinks.view(1, -1, 1, 1).to(torch.float32)
        new_max = torch.maximum(old_max, s)
        scale = torch.exp(old_max - new_max)
        w = w * scale
        den = den * scale + torch.exp(s - new_max)
    return (w / den).to(queries.dtype)


def apply_inv_mask_sum(input_tensor: torch.Tensor, mask: Mask) -> torch.Tensor:
    """Sum over the last dim of `mask.apply_inv_mask(input)`; plain sum for full/empty masks."""
    if tuple(input_tensor.shape) != tuple(mask.shape):
        raise ValueError(f"input_tensor.shape must be {mask.shape}, got {input_tensor.shape}")
    if mask.is_full or mask.is_empty:
        return input_tensor.sum(dim=-1, keepdim=True)
    return mask.apply_inv_mask(input_tensor).sum(dim=-1, keepdim=True)


def create_sampling_mask_with_per_head_budget(
    budgets: torch.Tensor,
    sampling_probability: torch.Tensor,
    seq_len_keys: int,
    start_idx: int,
    end_idx: int,
    dtype: torch.dtype = torch.float32,
) -> Mask:
    """Index-form mask with `budgets[row]` uniform draws (with replacement) per row.

    Reference: mask_attention_utils.py:105-184.  The draws come from
    `torch.randint` on the budgets' device, exactly one call of `sum(budgets)`
    elements, so a caller that seeds or replays that call gets the same mask.
    """
    b, h, q, _ = budgets.shape
    rows = b * h * q
    flat = budgets.reshape(rows)
    total = int(flat.sum().item())
    ptr = torch.zeros(rows + 1, dtype=torch.long, device=budgets.device)
    ptr[1:] = torch.cumsum(flat, dim=0)
    cols = torch.randint(low=start_idx, high=end_idx, size=(total,), device=budgets.device,
                         dtype=torch.long)
    row_id = torch.repeat_interleave(torch.arange(rows, device=budgets.device), flat.long(),
                                     output_size=total)
    data = sampling_probability.reshape(rows)[row_id]
    return Mask.create_mask_from_indices(shape=(b, h, q, seq_len_keys),
                                         indices=cols + row_id * seq_len_keys, ptr=ptr,
                                         data=data, dtype=dtype)


def get_attention_denominator(module, queries, keys, attention_mask, scaling, dropout,
                              sparse_attention_mask: Mask, **kwargs) -> torch.Tensor:
    training = module.training if module is not None else False
    w = _compute_masked_exp_attention_weights(queries, keys, attention_mask, scaling,
                                              sparse_attention_mask, dropout, training)
    return w.sum(dim=-1, keepdim=True)


def get_attention_numerator(module, queries, keys, values, attention_mask, scaling, dropout,
                            sparse_attention_mask: Mask, **kwargs) -> torch.Tensor:
    training = module.training if module is not None else False
    w = _compute_masked_exp_attention_weights(queries, keys, attention_mask, scaling,
                                              sparse_attention_mask, dropout, training)
    v = repeat_kv(values, _get_num_key_value_groups(queries, values)).to(torch.float32)
    return torch.matmul(w, v)


def get_true_attention_output(module, queries, keys, values, attention_mask, scaling, dropout,
                              **kwargs) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Dense SDPA over all keys, `[B, Sq, Hq, D]`; used by the output-error metric only."""
    groups = _get_num_key_value_groups(queries, keys)
    k, v = repeat_kv(keys, groups), repeat_kv(values, groups)
    am = attention_mask[:, :, :, : k.shape[-2]] if attention_mask is not None else None
    training = module.training if module is not None else False
    out = torch.nn.functional.scaled_dot_product_attention(
        query=queries, key=k, value=v, attn_mask=am, dropout_p=dropout if training else 0.0,
        is_causal=False, scale=scaling)
    return out.transpose(1, 2).contiguous(), None
