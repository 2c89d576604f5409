"""Thin Python wrappers around the C ABI, shared by the native maskers.

Each wrapper validates devices, allocates outputs with torch (device memory
and streams are torch's; all arithmetic is the library's) and launches on the
current CUDA stream of the tensors' device.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from .utils.mask import Mask, NativeBits, words_per_row


def _rows(shape: Sequence[int]) -> int:
    return int(np.prod(shape[:-1]))


def bias_args(attention_mask: Optional[torch.Tensor], dtype: torch.dtype, n_keys: int):
    """(keep-alive tensor, pointer, stride_b, stride_h, stride_q) for an additive bias."""
    from .utils.mask_attention_utils import _bias_args

    return _bias_args(attention_mask, dtype, n_keys)


def unit_weight_bits(previous_mask: Mask) -> Optional[NativeBits]:
    """Bitmap of `previous_mask` when all of its weights are 1, else None.

    Native maskers edit such bitmaps directly; a mask with other weights goes
    through its dense form instead.
    """
    if previous_mask.is_full:
        return None
    nb = previous_mask.native_bits()
    return nb if nb.data is None else None


def fresh_native(nb: NativeBits) -> NativeBits:
    """Same bitmap storage (and pending band edits), CSR companions dropped."""
    return nb.share()


def fill_band(nb: NativeBits, seq_len_queries: int, lo_base: int, lo_qstep: int, hi_base: int,
              hi_qstep: int, value: int) -> None:
    """Band edit of a unit-weight bitmap; applied with the next flush of its pending edits."""
    nb.add_band(seq_len_queries, lo_base, lo_qstep, hi_base, hi_qstep, value)


def bits_andnot(a: NativeBits, b: NativeBits) -> NativeBits:
    """a & ~b as a new bitmap (bookkeeping for the index-returning helper)."""
    return NativeBits(torch.bitwise_and(a.bits, torch.bitwise_not(b.bits)), a.rows, a.n_cols)


def topk_select(scores: torch.Tensor, previous_mask: Mask, k: int, col_begin: int = 0,
                col_end: Optional[int] = None, out: Optional[NativeBits] = None,
                per_row: bool = False) -> NativeBits:
    """previous | top-k of `scores` over inactive columns in [col_begin, col_end).

    `per_row`: one CTA per row in a single launch instead of rows spread over many CTAs with
    histograms in a scratch buffer; the better choice for many short rows (page scores)."""
    _native.require_cuda(scores, "scores")
    lib = _native.load()
    S = scores.shape[-1]
    rows = _rows(scores.shape)
    prev = previous_mask.native_bits()
    dst = out if out is not None else NativeBits(torch.empty_like(prev.bits), rows, S)
    sc = scores.contiguous()
    st = _native.stream_of(sc.device)
    end = S if col_end is None else col_end
    if rows <= 65535 and not per_row:
        # rows are spread over many CTAs; the histograms live in a scratch buffer
        nbytes = int(lib.sah_topk_select_ws_bytes(rows, prev.words))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=sc.device)
        _native.check(
            lib.sah_topk_select_ws(sc.data_ptr(), _native.dtype_code(sc.dtype), rows, S, prev.words,
                                   col_begin, end, prev.bits.data_ptr(), k, dst.bits.data_ptr(),
                                   ws.data_ptr(), nbytes, st), "sah_topk_select_ws")
        return dst
    _native.check(
        lib.sah_topk_select(sc.data_ptr(), _native.dtype_code(sc.dtype), rows, S, prev.words,
                            col_begin, end, prev.bits.data_ptr(), k, dst.bits.data_ptr(), st),
        "sah_topk_select")
    return dst


def topk_select_sharded(scores: torch.Tensor, previous_mask: Mask, k: int, comm, col_begin: int = 0,
                        col_end: Optional[int] = None) -> NativeBits:
    """`topk_select` when each row's keys are spread over the ranks of `comm` (contiguous ranges
    in rank order, `scores` holding this rank's columns): per digit of the radix select the
    ranks sum their 256-bin histograms, so all of them fix the same threshold; the count of
    keys equal to it is gathered and lower ranks are served first, which keeps the
    lowest-column tie rule.  `k` counts keys of the whole row.  Same result as the
    single-device selection, bit for bit."""
    _native.require_cuda(scores, "scores")
    lib = _native.load()
    S = scores.shape[-1]
    rows = _rows(scores.shape)
    if rows > 65535:
        raise NotImplementedError("sequence-sharded top-k handles at most 65535 mask rows per call")
    prev = previous_mask.native_bits()
    dst = NativeBits(torch.empty_like(prev.bits), rows, S)
    sc = scores.contiguous()
    dev = sc.device
    st = _native.stream_of(dev)
    code = _native.dtype_code(sc.dtype)
    end = S if col_end is None else col_end
    words = prev.words
    nbytes = int(lib.sah_topk_select_ws_bytes(rows, words))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    off = int(lib.sah_topk_sel_hist_offset(rows, words))
    hist = ws[off:off + rows * 1024].view(torch.int32)  # the digit histogram, summed in place
    _native.check(lib.sah_topk_sel_begin(rows, words, k, ws.data_ptr(), nbytes, st), "sah_topk_sel_begin")
    eq_total = torch.zeros(rows, dtype=torch.int64, device=dev)
    shifts = (8, 0) if sc.dtype == torch.bfloat16 else (24, 16, 8, 0)
    if k > 0:
        for shift in shifts:
            _native.check(lib.sah_topk_sel_hist(sc.data_ptr(), code, rows, S, words, col_begin, end,
                                                prev.bits.data_ptr(), ws.data_ptr(), shift, st),
                          "sah_topk_sel_hist")
            comm.all_reduce_sum_(hist)
            _native.check(lib.sah_topk_sel_pick(rows, words, ws.data_ptr(), shift, int(shift == shifts[0]),
                                                eq_total.data_ptr() if shift == 0 else None, st),
                          "sah_topk_sel_pick")
    gathered = comm.all_gather(eq_total)  # [world, rows]
    tie_offset = gathered[: comm.rank].sum(dim=0) if comm.rank > 0 else torch.zeros_like(eq_total)
    _native.check(lib.sah_topk_sel_emit(sc.data_ptr(), code, rows, S, words, col_begin, end,
                                        prev.bits.data_ptr(), ws.data_ptr(), tie_offset.data_ptr(),
                                        dst.bits.data_ptr(), st), "sah_topk_sel_emit")
    return dst


def qk_scores(queries: torch.Tensor, keys: torch.Tensor,
              attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
    """Unscaled q.k in the input dtype (+ additive bias), `[B, Hq, Sq, S]`."""
    _native.require_cuda(queries, "queries")
    _native.require_cuda(keys, "keys")
    lib = _native.load()
    B, Hq, Sq, D = queries.shape
    Hkv, S = keys.shape[1], keys.shape[2]
    q = queries if queries.stride(-1) == 1 else queries.contiguous()
    k = keys if keys.stride(-1) == 1 else keys.contiguous()
    scores = torch.empty((B, Hq, Sq, S), dtype=q.dtype, device=q.device)
    keep, bptr, bsb, bsh, bsq = bias_args(attention_mask, q.dtype, S)
    _native.check(
        lib.sah_qk_scores(q.data_ptr(), k.data_ptr(), _native.dtype_code(q.dtype), q.stride(0),
                          q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2), B, Hq,
                          Hkv, Sq, S, D, bptr, bsb, bsh, bsq, scores.data_ptr(),
                          _native.stream_of(q.device)),
        "sah_qk_scores")
    del keep
    return scores


def topp_select(scores: torch.Tensor, attention_mask: Optional[torch.Tensor], scaling: float,
                previous_mask: Mask, top_p: float, or_prev: bool) -> NativeBits:
    """Keys whose exp weight reaches the row's top-p threshold (`| previous` when `or_prev`).

    `scores` are the unscaled q.k of `qk_scores` without bias; bfloat16 only."""
    lib = _native.load()
    B, Hq, Sq, S = scores.shape
    prev = previous_mask.native_bits()
    dst = NativeBits(torch.empty_like(prev.bits), prev.rows, S)
    keep, bptr, bsb, bsh, bsq = bias_args(attention_mask, scores.dtype, S)
    table = exp_table(scores.device)
    _native.check(
        lib.sah_topp_select(scores.data_ptr(), _native.dtype_code(scores.dtype), float(scaling), bptr,
                            bsb, bsh, bsq, B, Hq, Sq, S, prev.words, prev.bits.data_ptr(), float(top_p),
                            table.data_ptr(), int(or_prev), dst.bits.data_ptr(),
                            _native.stream_of(scores.device)), "sah_topp_select")
    del keep
    return dst


# ---- HashAttention ------------------------------------------------------------
_ACT_TABLES: dict = {}


def _bf16_bits_to_f64(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def _f64_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16 (through float32, as a bf16 kernel does)."""
    f = x.astype(np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = rounded.astype(np.uint32) & 0xFFFF
    nan = np.isnan(f)
    out[nan] = 0x7FC0
    return out.astype(np.uint16)


def activation_table(name: str, device: torch.device) -> torch.Tensor:
    """uint16[65536]: bf16 bit pattern of x -> bf16 bit pattern of act(x).

    The activation is evaluated in float64 and rounded once to bfloat16, which
    is the value a float32 evaluation rounds to for every input except rare
    double-rounding cases.
    """
    key = (name, str(device))
    if key in _ACT_TABLES:
        return _ACT_TABLES[key]
    if name not in _native.ACTIVATIONS:
        raise ValueError(f"Unsupported activation function: {name}")
    bits = np.arange(65536, dtype=np.uint32)
    x = _bf16_bits_to_f64(bits)
    with np.errstate(over="ignore", invalid="ignore"):
        if name == "relu":
            y = np.maximum(x, 0.0)
        elif name == "silu":
            y = x / (1.0 + np.exp(-x))
        elif name == "gelu":
            from math import erf, sqrt
            y = 0.5 * x * (1.0 + np.vectorize(erf)(x / sqrt(2.0)))
        else:
            y = np.tanh(x)
    table = _f64_to_bf16_bits(np.where(np.isnan(x), x, y))
    t = torch.from_numpy(table.view(np.int16).copy()).to(device)
    _ACT_TABLES[key] = t
    return t


def hash_encode(x: torch.Tensor, n_heads_out: int, weights: List[torch.Tensor],
                biases: List[torch.Tensor], activation: str, codes: torch.Tensor,
                n_begin: int, n_end: int) -> None:
    """Pack sign(MLP(x[:, :, n_begin:n_end])) into `codes[:, :, n_begin:n_end]` (int32 words)."""
    _native.require_cuda(x, "hash input")
    lib = _native.load()
    B, H_in, _, D = x.shape
    xs = x if x.stride(-1) == 1 else x.contiguous()
    n_layers = len(weights)
    dims = [D] + [int(w.shape[-1]) for w in weights]
    for l, w in enumerate(weights):
        if tuple(w.shape) != (n_heads_out, dims[l], dims[l + 1]) or not w.is_contiguous():
            raise ValueError(f"hash weight {l} must be contiguous [H, {dims[l]}, {dims[l + 1]}]")
        if w.dtype != x.dtype or biases[l].dtype != x.dtype:
            raise ValueError("hash weights must be in the dtype of the hashed tensor")
    c_dims = (ctypes.c_int * len(dims))(*dims)
    c_w = (ctypes.c_void_p * n_layers)(*[w.data_ptr() for w in weights])
    c_b = (ctypes.c_void_p * n_layers)(*[b.data_ptr() for b in biases])
    table = activation_table(activation, x.device) if x.dtype == torch.bfloat16 else None
    _native.check(
        lib.sah_hash_encode(xs.data_ptr(), _native.dtype_code(x.dtype), xs.stride(0), xs.stride(1),
                            xs.stride(2), B, H_in, n_heads_out, n_begin, n_end, codes.shape[-1],
                            n_layers, c_dims, c_w, c_b, _native.ACTIVATIONS[activation],
                            _native.ptr(table), codes.data_ptr(), _native.stream_of(x.device)),
        "sah_hash_encode")


def hash_topk(kcodes: torch.Tensor, n_keys: int, qcodes: torch.Tensor, nbits: int,
              attention_mask: Optional[torch.Tensor], dtype: torch.dtype, previous_mask: Mask,
              k: int, shape: Tuple[int, int, int, int]) -> NativeBits:
    """previous | top-k Hamming matches; kcodes `[B, Hq, capacity]` with `n_keys` valid."""
    lib = _native.load()
    B, Hq, Sq, S = shape
    if kcodes.shape[-1] < S or not kcodes.is_contiguous():
        raise ValueError("key codes must be contiguous [B, Hq, capacity >= S]")
    prev = previous_mask.native_bits()
    dst = NativeBits(torch.empty_like(prev.bits), prev.rows, S)
    dev = kcodes.device
    st = _native.stream_of(dev)
    sms = _native.sm_count(dev)
    if attention_mask is None and (prev.rows < sms or prev.words > 2048):
        # fewer rows than SMs (long contexts, small batches), or rows too long for the
        # register-resident kernel: histogram, then emit, with every row cut into chunks so
        # that the grid fills the device; otherwise the one-CTA-per-row kernel below does the
        # same in a single launch
        nbytes = int(lib.sah_hash_topk_ws_bytes(prev.rows, prev.words, sms))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _native.check(
            lib.sah_hash_topk_ws(kcodes.data_ptr(), kcodes.shape[-1], qcodes.data_ptr(), nbits, B, Hq, Sq,
                                 S, prev.words, prev.bits.data_ptr(), k, dst.bits.data_ptr(),
                                 ws.data_ptr(), nbytes, sms, st), "sah_hash_topk_ws")
        return dst
    keep, bptr, bsb, bsh, bsq = bias_args(attention_mask, dtype, S)
    _native.check(
        lib.sah_hash_topk(kcodes.data_ptr(), kcodes.shape[-1], qcodes.data_ptr(), nbits, bptr,
                          _native.dtype_code(dtype), bsb, bsh, bsq, B, Hq, Sq, S, prev.words,
                          prev.bits.data_ptr(), k, dst.bits.data_ptr(), st),
        "sah_hash_topk")
    del keep
    return dst


def hash_topk_sharded(kcodes: torch.Tensor, qcodes: torch.Tensor, nbits: int, previous_mask: Mask,
                      k: int, shape: Tuple[int, int, int, int], comm) -> NativeBits:
    """`hash_topk` when the row's keys are spread over the ranks of `comm` (contiguous ranges in
    rank order): local histogram, one all-gather of `rows x 33` counters, global threshold
    with the ties served to the lowest columns first, local emit.  `k` counts keys of the
    whole sequence; `shape[-1]` is the local key count."""
    lib = _native.load()
    B, Hq, Sq, S = shape
    if kcodes.shape[-1] < S or not kcodes.is_contiguous():
        raise ValueError("key codes must be contiguous [B, Hq, capacity >= S]")
    dev = kcodes.device
    st = _native.stream_of(dev)
    prev = previous_mask.native_bits()
    rows = prev.rows
    # every rank cuts its range into the same number of chunks (one CTA per row and chunk);
    # the count depends on the row count only, so that all ranks agree on it
    words = prev.words
    chunks = max(1, min(-(-_native.sm_count(dev) * 8 // rows), 256))
    hist = torch.empty((chunks, rows, 33), dtype=torch.int32, device=dev)
    args = (kcodes.data_ptr(), kcodes.shape[-1], qcodes.data_ptr(), nbits, B, Hq, Sq, S, words, chunks,
            prev.bits.data_ptr())
    # one byte per key carries the scores from the histogram pass to the emit pass
    scores = torch.empty(int(lib.sah_hash_scores_bytes(rows, words)), dtype=torch.uint8, device=dev)
    _native.check(lib.sah_hash_hist(*args, hist.data_ptr(), scores.data_ptr(), st), "sah_hash_hist")
    hist_all = comm.all_gather(hist)  # [world, chunks, rows, 33]
    thr = torch.empty((chunks, rows), dtype=torch.int32, device=dev)
    need = torch.empty((chunks, rows), dtype=torch.int64, device=dev)
    _native.check(lib.sah_hash_shard_plan(hist_all.data_ptr(), comm.world, comm.rank, chunks, rows, k,
                                          thr.data_ptr(), need.data_ptr(), st), "sah_hash_shard_plan")
    dst = NativeBits(torch.empty_like(prev.bits), rows, S)
    _native.check(lib.sah_hash_emit(*args, thr.data_ptr(), need.data_ptr(), scores.data_ptr(),
                                    dst.bits.data_ptr(), st), "sah_hash_emit")
    return dst


# ---- sampled sets ---------------------------------------------------------------
def merge_sampled(previous_mask: Mask, cols: torch.Tensor, sptr: torch.Tensor,
                  row_weight: torch.Tensor) -> Mask:
    """`clamp(previous + sampled, 0, 1)` (Mask.merge_mask_dense) for a ragged sample list.

    `cols` int64 [n] are key columns, sample j belongs to the row r with
    sptr[r] <= j < sptr[r+1]; every sampled position carries `row_weight[row]`
    (mask dtype).  Duplicates collapse to one entry; a position already active in the
    previous (unit-weight) mask keeps weight 1.  No host synchronisation: the weight
    array is sized for the worst case and the CSR pointers stay on the device.
    """
    _native.require_cuda(cols, "sampled columns")
    lib = _native.load()
    shape = tuple(previous_mask.shape)
    S = shape[-1]
    rows = _rows(shape)
    dev = cols.device
    st = _native.stream_of(dev)
    dtype = previous_mask.dtype
    prev = unit_weight_bits(previous_mask)
    words = words_per_row(S)
    samp = torch.zeros((rows, words), dtype=torch.int32, device=dev)
    cols = cols.contiguous()
    sptr = sptr.to(torch.int64).contiguous()
    _native.check(lib.sah_mask_scatter_samples(cols.data_ptr(), sptr.data_ptr(), rows, cols.numel(), S,
                                               words, samp.data_ptr(), st), "sah_mask_scatter_samples")
    return merge_sampled_bits(previous_mask, samp, row_weight, cols.numel())


def merge_sampled_bits(previous_mask: Mask, samp: torch.Tensor, row_weight: torch.Tensor,
                       n_samples_bound: int) -> Mask:
    """Second half of `merge_sampled`: the sampled set is already a bitmap `[rows, W]`."""
    lib = _native.load()
    shape = tuple(previous_mask.shape)
    S = shape[-1]
    rows = _rows(shape)
    dev = samp.device
    st = _native.stream_of(dev)
    dtype = previous_mask.dtype
    prev = unit_weight_bits(previous_mask)
    words = samp.shape[-1]
    if prev is None:
        # weighted (or full) previous mask: the general dense merge
        add = Mask._from_native(shape, dtype, _sampled_native(samp, None, rows, S, words, row_weight,
                                                              dtype, n_samples_bound))
        return previous_mask.merge_mask(add, inplace=False)
    merged = torch.empty_like(samp)
    _native.check(lib.sah_mask_or(prev.bits.data_ptr(), samp.data_ptr(), rows * words,
                                  merged.data_ptr(), st), "sah_mask_or")
    # the number of entries is only known on the device: size the weights for the worst case
    nb = _sampled_native(merged, prev.bits, rows, S, words, row_weight, dtype, rows * S)
    return Mask._from_native(shape, dtype, nb)


_EXP_TABLES: dict = {}


def exp_table(device: torch.device) -> torch.Tensor:
    """uint16[65536]: bf16 bit pattern of x -> bf16 bit pattern of exp(x) (float64 evaluation,
    rounded through float32), for kernels that reproduce a bf16 `torch.exp`."""
    key = str(device)
    if key not in _EXP_TABLES:
        x = _bf16_bits_to_f64(np.arange(65536, dtype=np.uint32))
        with np.errstate(over="ignore", invalid="ignore"):
            y = np.exp(x)
        table = _f64_to_bf16_bits(np.where(np.isnan(x), x, y))
        _EXP_TABLES[key] = torch.from_numpy(table.view(np.int16).copy()).to(device)
    return _EXP_TABLES[key]


def _sampled_native(bits: torch.Tensor, prev_bits: Optional[torch.Tensor], rows: int, S: int,
                    words: int, row_weight: torch.Tensor, dtype: torch.dtype,
                    nnz_bound: int) -> NativeBits:
    lib = _native.load()
    dev = bits.device
    st = _native.stream_of(dev)
    nb = NativeBits(bits, rows, S)
    nb.ensure_scan()
    data = torch.empty(min(nnz_bound, rows * S), dtype=dtype, device=dev)
    rw = row_weight.to(dtype).reshape(rows).contiguous()
    _native.check(
        lib.sah_mask_sample_data(_native.ptr(prev_bits), bits.data_ptr(), nb.wpre.data_ptr(),
                                 nb.ptr.data_ptr(), rw.data_ptr(), None, _native.dtype_code(dtype),
                                 rows, S, words, data.data_ptr(), st), "sah_mask_sample_data")
    nb.data = data
    return nb


# ---- merge of two bitmap-form masks -------------------------------------------------
def _side(nb: NativeBits):
    if nb.data is not None:
        nb.ensure_scan()
        return (nb.bits.data_ptr(), nb.data.data_ptr(), nb.wpre.data_ptr(), nb.ptr.data_ptr())
    return (nb.bits.data_ptr(), None, None, None)


def merge_native(a: Mask, b: Mask) -> Mask:
    """`clamp(a + b, 0, 1)` (Mask.merge_mask_dense, utils/mask.py:875-877) on the bitmap
    forms of two masks that are neither full nor empty.  No dense tensor is built and
    nothing is read back: the weight array is sized for the worst case."""
    lib = _native.load()
    an, bn = a.native_bits(), b.native_bits()
    dev = an.bits.device
    st = _native.stream_of(dev)
    rows, S, W = an.rows, an.n_cols, an.words
    code = _native.dtype_code(a.dtype)
    out_bits = torch.empty_like(an.bits)
    sa, sb = _side(an), _side(bn)
    _native.check(lib.sah_mask_merge_bits(*sa, *sb, code, rows, W, out_bits.data_ptr(), st),
                  "sah_mask_merge_bits")
    nb = NativeBits(out_bits, rows, S)
    if an.data is not None or bn.data is not None:
        nb.ensure_scan()
        bound = rows * S
        if an.data is not None and bn.data is not None:
            bound = min(bound, an.data.numel() + bn.data.numel())
        data = torch.empty(bound, dtype=a.dtype, device=dev)
        _native.check(
            lib.sah_mask_merge_data(*sa, *sb, code, rows, W, out_bits.data_ptr(), nb.wpre.data_ptr(),
                                    nb.ptr.data_ptr(), data.data_ptr(), st), "sah_mask_merge_data")
        nb.data = data
    return Mask._from_native(tuple(a.shape), a.dtype, nb)


# ---- bounded device-side waits ------------------------------------------------------
def wait_errors() -> int:
    """How many attention workspaces carry a set error word: a bounded wait of the tensor-map
    copy stage ran out in some launch that used them and its result is incomplete (reads
    device memory: synchronises)."""
    from .utils import mask_attention_utils as mau

    return mau.attention_wait_errors()


# ---- MagicPig ---------------------------------------------------------------------
_LSH_TABLES: dict = {}


def lsh_weight_table(device: torch.device, lsh_k: int, lsh_l: int) -> torch.Tensor:
    """uint16[65536]: bf16 bits of a cosine -> bf16 bits of the sampling weight 1 / (p + 1e-6) of
    its collision probability p (`lsh_prob_table`), rounded as Mask.apply_inv_mask_dense rounds it
    in bfloat16 (utils/mask.py:718-740: the sum to bf16, the reciprocal to bf16); 0 where p is 0
    (a zero in the reference's dense mask means "not selected")."""
    key = (str(device), lsh_k, lsh_l, "weight")
    if key not in _LSH_TABLES:
        pbits = lsh_prob_table(torch.device("cpu"), lsh_k, lsh_l).numpy().view(np.uint16).astype(np.uint32)
        p = (pbits << 16).view(np.float32)
        with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
            s = _bf16_bits_to_f64(_f64_to_bf16_bits((p + np.float32(1e-6)).astype(np.float64))).astype(np.float32)
            w = _f64_to_bf16_bits((np.float32(1.0) / s).astype(np.float64))
        w = np.where(p == 0.0, np.uint16(0), w.astype(np.uint16)).astype(np.uint16)
        _LSH_TABLES[key] = torch.from_numpy(w.view(np.int16).copy()).to(device)
    return _LSH_TABLES[key]


def lsh_prob_table(device: torch.device, lsh_k: int, lsh_l: int) -> torch.Tensor:
    """uint16[65536]: bf16 bits of a cosine -> bf16 bits of the collision probability
    1 - (1 - (1 - acos(c)/pi)^K)^L with every operation rounded to bf16 as a bf16 tensor
    program rounds it (magic_pig.py:389-403); float64 evaluation rounded through float32."""
    key = (str(device), lsh_k, lsh_l)
    if key not in _LSH_TABLES:
        bf = lambda x: _bf16_bits_to_f64(_f64_to_bf16_bits(x))  # noqa: E731
        with np.errstate(invalid="ignore", over="ignore"):
            c = _bf16_bits_to_f64(np.arange(65536, dtype=np.uint32))
            c = np.clip(c, -1.0, 1.0)  # NaN stays NaN
            theta = bf(np.arccos(c))
            a = bf((theta.astype(np.float32) / np.float32(np.pi)).astype(np.float64))
            s = bf(1.0 - a)
            st = bf(np.power(s, float(lsh_k)))
            u = bf(1.0 - st)
            ul = bf(np.power(u, float(lsh_l)))
            table = _f64_to_bf16_bits(1.0 - ul)
        _LSH_TABLES[key] = torch.from_numpy(table.view(np.int16).copy()).to(device)
    return _LSH_TABLES[key]
