"""CUDA path vs the numpy restatement and vs the reference's golden outputs.

Every call goes through the Python API, which reaches the kernels through the
C ABI of libsah_b200.so.  Index sets, ptr arrays, mask weights and integer
codes must be bit-exact; attention outputs within 1e-4 (fp32) / 2e-2 (bf16),
absolute and relative.
"""

import numpy as np
import pytest
import torch

from oracle import attention as o_attention
from oracle import hashattention as o_hash
from oracle import mask_ops, qk as o_qk, stacks
import workloads
from sparse_attention_hub.sparse_attention import Mask
from sparse_attention_hub.sparse_attention import _native_ops
from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import (
    get_masked_attention_output,
    native_masked_attention,
)

from conftest import load_golden

pytestmark = pytest.mark.gpu
TOL = {"f32": 1e-4, "bf16": 2e-2}
DEV = "cuda:0"


def _run_native(wl, attention_mask=None, sinks=None, meta=None):
    ra = workloads.research_attention(wl.stack, wl.dtype, DEV)
    q, k, v = (workloads.to_torch(a, wl.dtype, DEV) for a in (wl.q, wl.k, wl.v))
    am = None if attention_mask is None else workloads.to_torch(attention_mask, wl.dtype, DEV)
    meta = {} if meta is None else meta
    mask = ra.build_mask(q, k, v, am, float(wl.scaling), 0.0, meta, layer_idx=0)
    s = None if sinks is None else torch.from_numpy(sinks).to(DEV)
    out = get_masked_attention_output(None, q, k, v, am, s, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    return mask, out.float().cpu().numpy(), meta


def _assert_mask_equal(mask: Mask, ref_dense=None, golden=None):
    idx, ptr, data = mask.get_index_mask()
    idx, ptr, data = idx.cpu().numpy(), ptr.cpu().numpy(), data.float().cpu().numpy()
    if ref_dense is not None:
        ri, rp, rd = mask_ops.to_csr(ref_dense)
        np.testing.assert_array_equal(idx, ri)
        np.testing.assert_array_equal(ptr, rp)
        np.testing.assert_array_equal(data, rd)
    if golden is not None:
        np.testing.assert_array_equal(idx, golden["idx"])
        np.testing.assert_array_equal(ptr, golden["ptr"])
        np.testing.assert_array_equal(data, golden["data"])


def _close(a, b, dtype, scale=1.0):
    np.testing.assert_allclose(a, b, atol=TOL[dtype] * scale, rtol=TOL[dtype] * scale)


# ---------------------------------------------------------------------------
def test_sink_local_f32_golden_and_oracle():
    g = load_golden("sink_local_f32")
    wl = workloads.sink_local_fp32(seed=11, B=1, Hq=8, Hkv=2, S=640, D=128, sink=16, window=48)
    mask, out, _ = _run_native(wl)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "f32")
    _assert_mask_equal(mask, ref_mask, g)
    _close(out, ref_out, "f32")
    _close(out, g["out"], "f32")


def test_sink_local_sq3_causal_sinks():
    g = load_golden("sink_local_f32_sq3_causal_sinks")
    wl = workloads.sink_local_fp32(seed=12, B=2, Hq=4, Hkv=2, S=320, D=64, sink=8, window=24, Sq=3)
    mask, out, _ = _run_native(wl, attention_mask=g["attention_mask"], sinks=g["sinks"])
    _assert_mask_equal(mask, golden=g)
    _close(out, g["out"], "f32")


def test_sink_local_bf16_fraction():
    g = load_golden("sink_local_bf16_fraction")
    wl = workloads.sink_local_fp32(seed=13, B=2, Hq=8, Hkv=4, S=512, D=128)
    wl.dtype = "bf16"
    wl.q, wl.k, wl.v = (workloads.to_dtype(a, "bf16") for a in (wl.q, wl.k, wl.v))
    wl.stack = [("sink", {"sink_size": 0.05}), ("local", {"window_size": 0.1})]
    mask, out, _ = _run_native(wl)
    _assert_mask_equal(mask, golden=g)
    _close(out, g["out"], "bf16")


def test_cpu_runnable_config_full_size():
    """Sink(128)+Local(256), fp32, S=4096, 32/8 heads: the first benchmark configuration."""
    wl = workloads.sink_local_fp32(seed=1)
    mask, out, _ = _run_native(wl)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "f32")
    _assert_mask_equal(mask, ref_mask)
    _close(out, ref_out, "f32")


# ---------------------------------------------------------------------------
def test_hash_codes_bit_exact_vs_oracle_and_golden():
    g = load_golden("hash_bf16")
    wl = workloads.hashattention_bf16(seed=21, B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16, window=32)
    mask, out, meta = _run_native(wl)
    kc = meta["key"][0]
    codes = kc.codes[..., : kc.length].cpu().numpy().view(np.uint32)
    w = wl.stack[2][1]["weights"]
    ref_codes = o_hash.signatures(o_attention.repeat_kv(wl.k, 4), w["key_matrix"], w["key_bias"],
                                  "silu", "bf16")
    np.testing.assert_array_equal(codes, ref_codes)
    np.testing.assert_array_equal(codes, g["kcodes"])  # the reference's own bits
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16")
    _assert_mask_equal(mask, ref_mask, g)
    _close(out, ref_out, "bf16")
    _close(out, g["out"], "bf16")


@pytest.mark.parametrize("act", ["relu", "gelu", "tanh"])
def test_hash_other_activations(act):
    wl = workloads.hashattention_bf16(seed=22, B=1, Hq=4, Hkv=2, S=777, D=128, sink=4, window=9,
                                      heavy=40, bits=32, hidden=64, layers=2, activation=act)
    mask, out, _ = _run_native(wl)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16")
    _assert_mask_equal(mask, ref_mask)
    _close(out, ref_out, "bf16")


def test_hash_incremental_key_cache():
    """Keys appended between calls are hashed incrementally and give the same codes."""
    wl = workloads.hashattention_bf16(seed=23, B=1, Hq=8, Hkv=2, S=900, D=128, sink=8, window=16)
    ra = workloads.research_attention(wl.stack, "bf16", DEV)
    q, k, v = (workloads.to_torch(a, "bf16", DEV) for a in (wl.q, wl.k, wl.v))
    meta = {}
    ra.build_mask(q, k[:, :, :600], v[:, :, :600], None, wl.scaling, 0.0, meta, layer_idx=0)
    m2 = ra.build_mask(q, k, v, None, wl.scaling, 0.0, meta, layer_idx=0)
    fresh = ra.build_mask(q, k, v, None, wl.scaling, 0.0, {}, layer_idx=0)
    a, b = m2.get_index_mask(), fresh.get_index_mask()
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    # and both are what the restatement selects on all 900 keys
    ref_mask, _, rmeta = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16")
    _assert_mask_equal(m2, ref_mask)
    kc = meta["key"][0]
    np.testing.assert_array_equal(kc.codes[..., : kc.length].cpu().numpy().view(np.uint32), rmeta["hash_kcodes"])
    with pytest.raises(ValueError):
        ra.build_mask(q, k[:, :, :100], v[:, :, :100], None, wl.scaling, 0.0, meta, layer_idx=0)


def test_hash_with_attention_mask_blocking_keys():
    wl = workloads.hashattention_bf16(seed=24, B=2, Hq=4, Hkv=2, S=640, D=128, sink=8, window=16,
                                      heavy=64)
    am = np.zeros((2, 1, 1, 640), np.float32)
    am[0, :, :, 100:300] = -3.3895313892515355e38  # padded positions of batch 0
    mask, out, _ = _run_native(wl, attention_mask=am)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                            attention_mask=am)
    _assert_mask_equal(mask, ref_mask)
    _close(out, ref_out, "bf16")


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,seed", [("bf16", 31), ("f32", 32)])
def test_oracle_topk(dtype, seed):
    g = load_golden(f"oracle_topk_{dtype}")
    wl = workloads.oracle_topk(seed=seed, dtype=dtype, B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16,
                               window=32, heavy=0.02)
    mask, out, _ = _run_native(wl)
    ref_mask, ref_out, rmeta = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype)
    # scores bit-exact against the restatement's fixed summation order
    q, k = (workloads.to_torch(a, dtype, DEV) for a in (wl.q, wl.k))
    s = _native_ops.qk_scores(q, k, None).float().cpu().numpy()
    np.testing.assert_array_equal(s, rmeta["oracle_scores"])
    _assert_mask_equal(mask, ref_mask)
    _close(out, ref_out, dtype)
    _close(out, g["out"], dtype, scale=2.0)
    # selection kernel on the reference's own score tensor reproduces its mask exactly
    prev = workloads.research_attention(wl.stack[:2], dtype, DEV).build_mask(
        q, k, k, None, wl.scaling, 0.0, {}, layer_idx=0)
    sc = workloads.to_torch(g["scores"], dtype, DEV)
    sel = _native_ops.topk_select(sc, prev, int(0.02 * 1024))
    _assert_mask_equal(Mask._from_native(tuple(sc.shape), workloads.torch_dtype(dtype), sel), golden=g)


def test_topk_select_ties_and_short_rows():
    S = 1000
    sc = torch.zeros((1, 3, 1, S), device=DEV)           # all equal: lowest columns win
    sc[0, 1, 0, 500:] = 1.0
    sc[0, 2, 0, ::7] = -0.0
    prev = Mask.create_empty_mask((1, 3, 1, S), torch.float32, torch.device(DEV))
    sel = Mask._from_native((1, 3, 1, S), torch.float32, _native_ops.topk_select(sc, prev, 37))
    dense = sel.get_dense_mask().cpu().numpy()[0, :, 0]
    assert dense[0, :37].all() and dense[0].sum() == 37
    assert dense[1, 500:537].all() and dense[1].sum() == 37
    assert dense[2, :37].all() and dense[2].sum() == 37
    everything = _native_ops.topk_select(sc, prev, 5000)  # k beyond the row: every candidate
    assert Mask._from_native((1, 3, 1, S), torch.float32, everything).get_density() == 1.0


@pytest.mark.parametrize("dtype,S,rows_h,k", [("bf16", 512, 40, 25), ("f32", 700, 9, 60), ("bf16", 5000, 5, 333),
                                              ("f32", 33, 3, 40)])
def test_topk_select_one_cta_per_row_equals_chunked(dtype, S, rows_h, k):
    """Both exact top-k paths give the same bitmap, previous mask and ties included."""
    rng = np.random.default_rng(S + k)
    x = rng.normal(size=(1, rows_h, 1, S)).astype(np.float32)
    x[0, 0, 0, : S // 2] = np.round(x[0, 0, 0, : S // 2])       # many ties
    sc = workloads.to_torch(workloads.to_dtype(x, dtype), dtype, DEV)
    shape = (1, rows_h, 1, S)
    prev_np = np.zeros(shape, np.float32)
    prev_np[..., :5] = 1.0
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    prev = Mask.create_mask_from_dense_mask(shape, torch.from_numpy(prev_np).to(DEV).to(tdt), tdt)
    a = _native_ops.topk_select(sc, prev, k)
    b = _native_ops.topk_select(sc, prev, k, per_row=True)
    assert torch.equal(a.bits, b.bits)
    from oracle import topk as ot
    want = ot.topk_inactive(sc.float().cpu().numpy(), prev_np != 0, k) | (prev_np != 0)
    got = Mask._from_native(shape, tdt, b).get_dense_mask().float().cpu().numpy() != 0
    np.testing.assert_array_equal(got, want)


# ---------------------------------------------------------------------------
def test_mask_conversions_round_trip():
    rng = np.random.default_rng(5)
    dense = (rng.random((2, 3, 2, 333)) < 0.2) * rng.random((2, 3, 2, 333))
    dense = workloads.to_dtype(dense.astype(np.float32), "bf16")
    t = workloads.to_torch(dense, "bf16", DEV)
    m = Mask.create_mask_from_dense_mask(t.shape, t, torch.bfloat16)
    idx, ptr, data = m.get_index_mask()
    ri, rp, rd = mask_ops.to_csr(dense)
    np.testing.assert_array_equal(idx.cpu().numpy(), ri)
    np.testing.assert_array_equal(ptr.cpu().numpy(), rp)
    np.testing.assert_array_equal(data.float().cpu().numpy(), rd)
    nb = m.native_bits()
    back = Mask._from_native(tuple(t.shape), torch.bfloat16, nb).get_dense_mask()
    assert torch.equal(back, t)


def test_weighted_mask_attention_matches_oracle():
    """Non-unit weights (sampling probabilities) enter numerator and denominator."""
    wl = workloads.sink_local_fp32(seed=41, B=2, Hq=8, Hkv=2, S=700, D=128)
    rng = np.random.default_rng(7)
    for dtype in ("f32", "bf16"):
        q, k, v = (workloads.to_dtype(a, dtype) for a in (wl.q, wl.k, wl.v))
        dense = np.where(rng.random((2, 8, 1, 700)) < 0.15, rng.uniform(0.05, 1.0, (2, 8, 1, 700)), 0.0)
        dense[..., :8] = 1.0
        dense = workloads.to_dtype(dense.astype(np.float32), dtype)
        tq, tk, tv = (workloads.to_torch(a, dtype, DEV) for a in (q, k, v))
        m = Mask.create_mask_from_dense_mask(dense.shape, workloads.to_torch(dense, dtype, DEV),
                                             workloads.torch_dtype(dtype))
        out = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), m)
        ref = o_attention.masked_attention(q, k, v, dense, wl.scaling, dtype)
        _close(out.float().cpu().numpy(), ref, dtype)


def test_full_and_empty_masks_mean_dense_attention():
    wl = workloads.sink_local_fp32(seed=42, B=1, Hq=8, Hkv=8, S=300, D=64)
    tq, tk, tv = (workloads.to_torch(a, "f32", DEV) for a in (wl.q, wl.k, wl.v))
    ref = o_attention.masked_attention(wl.q, wl.k, wl.v, None, wl.scaling, "f32", no_mask=True)
    for m in (Mask.create_full_mask((1, 8, 1, 300), torch.float32, torch.device(DEV)),
              Mask.create_empty_mask((1, 8, 1, 300), torch.float32, torch.device(DEV))):
        out = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), m)
        _close(out.cpu().numpy(), ref, "f32")


def test_partials_merge_equals_single_pass():
    """Sequence-sharded partials merged by the merge kernel equal the one-shot result."""
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import merge_attention_partials

    wl = workloads.sink_local_fp32(seed=43, B=1, Hq=8, Hkv=2, S=1024, D=128, sink=32, window=64)
    tq, tk, tv = (workloads.to_torch(a, "f32", DEV) for a in (wl.q, wl.k, wl.v))
    rng = np.random.default_rng(3)
    dense = (rng.random((1, 8, 1, 1024)) < 0.1).astype(np.float32)
    full = Mask.create_mask_from_dense_mask(dense.shape, torch.from_numpy(dense).to(DEV), torch.float32)
    want = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), full)
    parts = []
    for lo, hi in ((0, 512), (512, 1024)):
        part = Mask.create_mask_from_dense_mask((1, 8, 1, hi - lo),
                                                torch.from_numpy(dense[..., lo:hi].copy()).to(DEV),
                                                torch.float32)
        _, p = native_masked_attention(tq, tk[:, :, lo:hi].contiguous(),
                                       tv[:, :, lo:hi].contiguous(), None, None,
                                       float(wl.scaling), part, return_partials=True)
        parts.append(p)
    got = merge_attention_partials(torch.stack(parts), 1, 8, 1, torch.float32)
    _close(got.cpu().numpy(), want.cpu().numpy(), "f32")
    # and the restatement's dense computation over all keys
    ref = o_attention.masked_attention(wl.q, wl.k, wl.v, dense, wl.scaling, "f32")
    _close(got.cpu().numpy(), ref, "f32")


def test_hash_topk_degenerate_score_distributions():
    """Rows whose scores are nothing like a binomial: all equal, two levels, all maximal."""
    S, k = 5000, 300
    shape = (1, 4, 1, S)
    rng = np.random.default_rng(9)
    q = np.array([[[0x0F0F0F0F], [0xFFFFFFFF], [0x12345678], [0]]], np.uint32)
    kc = np.empty((1, 4, S), np.uint32)
    kc[0, 0] = ~q[0, 0, 0]                      # every key scores 0 matching bits
    kc[0, 1] = q[0, 1, 0]                       # every key matches all 32 bits
    kc[0, 2] = np.where(rng.random(S) < 0.01, q[0, 2, 0], ~q[0, 2, 0])  # 1 % perfect, rest zero
    kc[0, 3] = rng.integers(0, 2 ** 32, S, dtype=np.uint64).astype(np.uint32)
    tk = torch.from_numpy(kc.view(np.int32)).to(DEV)
    tq = torch.from_numpy(q.view(np.int32)).to(DEV)
    prev = Mask.create_empty_mask(shape, torch.bfloat16, torch.device(DEV))
    sel = _native_ops.hash_topk(tk, S, tq, 32, None, torch.bfloat16, prev, k, shape)
    got = Mask._from_native(shape, torch.bfloat16, sel).get_dense_mask().float().cpu().numpy() != 0
    from oracle import hashattention as oh, topk as ot
    scores = oh.scores(q, kc, 32, "bf16")
    want = ot.topk_inactive(scores, np.zeros(shape, bool), k)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("S,cap,rows_h,k,nbits,path", [
    (5000, 5003, 4, 300, 32, "row"),      # ragged tail, odd capacity: rows 1.. are not 16-byte aligned
    (5000, 5003, 4, 300, 32, "chunks"),
    (16384, 16384, 3, 512, 32, "row"),    # one word per thread
    (40000, 40960, 2, 1000, 16, "row"),   # two / four words per thread, 16-bit codes
    (40000, 40960, 2, 1000, 16, "chunks"),
    (70001, 70016, 2, 4000, 32, "row"),   # longer than the register-resident kernel takes
    (70001, 70016, 2, 4000, 32, "chunks"),
    (300000, 300000, 1, 9000, 32, "chunks"),
    (300000, 300000, 2, 9000, 32, "pieces"),  # two chunks per row: the byte counters flush several times
    (300000, 300000, 2, 9000, 32, "pieces_scratch"),  # the same with the one-byte score scratch
    (1500, 1500, 2, 0, 32, "row"),
    (1500, 1500, 2, 5000, 32, "chunks"),  # k above the number of candidates
])
def test_hash_topk_kernel_variants(S, cap, rows_h, k, nbits, path):
    """Every Hamming top-k kernel (one CTA per row: register-resident and streaming; chunked
    rows with the plan fused into the emit pass) against the same selection rule, with a
    previous mask in place and score ties cut in column order."""
    from oracle import hashattention as oh, topk as ot
    from sparse_attention_hub import _native
    lib = _native.load()
    rng = np.random.default_rng(S + k + nbits)
    shape = (1, rows_h, 1, S)
    mask_bits = np.uint64((1 << nbits) - 1)
    kc = np.zeros((1, rows_h, cap), np.uint32)
    kc[..., :S] = (rng.integers(0, 2 ** 32, (1, rows_h, S), dtype=np.uint64) & mask_bits).astype(np.uint32)
    kc[0, 0, : S // 2] &= np.uint32(0xFF)   # a row with few distinct scores: long tie runs
    q = (rng.integers(0, 2 ** 32, (1, rows_h, 1), dtype=np.uint64) & mask_bits).astype(np.uint32)
    prev_np = np.zeros(shape, bool)
    prev_np[..., :37] = True
    prev_np[..., S - 70:] = True
    prev_np[0, 0, 0, rng.integers(0, S, 200)] = True
    prev = Mask.create_mask_from_dense_mask(shape, torch.from_numpy(prev_np).to(DEV).to(torch.bfloat16),
                                            torch.bfloat16)
    pb = prev.native_bits()
    tk = torch.from_numpy(kc.view(np.int32)).to(DEV)
    tq = torch.from_numpy(q.view(np.int32)).to(DEV)
    out = torch.empty_like(pb.bits)
    st = _native.stream_of(tk.device)
    if path == "row":
        _native.check(lib.sah_hash_topk(tk.data_ptr(), cap, tq.data_ptr(), nbits, None, _native.SAH_BF16, 0, 0, 0,
                                        1, rows_h, 1, S, pb.words, pb.bits.data_ptr(), k, out.data_ptr(), st),
                      "sah_hash_topk")
    elif path in ("pieces", "pieces_scratch"):
        chunks = 2
        scratch = None
        if path == "pieces_scratch":
            scratch = torch.empty(int(lib.sah_hash_scores_bytes(pb.rows, pb.words)), dtype=torch.uint8, device=DEV)
        sp = None if scratch is None else scratch.data_ptr()
        hist = torch.empty((chunks, pb.rows, 33), dtype=torch.int32, device=DEV)
        thr = torch.empty((chunks, pb.rows), dtype=torch.int32, device=DEV)
        need = torch.empty((chunks, pb.rows), dtype=torch.int64, device=DEV)
        args = (tk.data_ptr(), cap, tq.data_ptr(), nbits, 1, rows_h, 1, S, pb.words, chunks, pb.bits.data_ptr())
        _native.check(lib.sah_hash_hist(*args, hist.data_ptr(), sp, st), "sah_hash_hist")
        _native.check(lib.sah_hash_shard_plan(hist.data_ptr(), 1, 0, chunks, pb.rows, k, thr.data_ptr(),
                                              need.data_ptr(), st), "sah_hash_shard_plan")
        _native.check(lib.sah_hash_emit(*args, thr.data_ptr(), need.data_ptr(), sp, out.data_ptr(), st),
                      "sah_hash_emit")
    else:
        sms = _native.sm_count(tk.device)
        nbytes = int(lib.sah_hash_topk_ws_bytes(pb.rows, pb.words, sms))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
        _native.check(lib.sah_hash_topk_ws(tk.data_ptr(), cap, tq.data_ptr(), nbits, 1, rows_h, 1, S, pb.words,
                                           pb.bits.data_ptr(), k, out.data_ptr(), ws.data_ptr(), nbytes, sms,
                                           st), "sah_hash_topk_ws")
    got = Mask._from_native(shape, torch.bfloat16, type(pb)(out, pb.rows, S)).get_dense_mask().float().cpu().numpy() != 0
    scores = oh.scores(q, kc[..., :S], nbits, "bf16")
    want = ot.topk_inactive(scores, prev_np, k) | prev_np
    np.testing.assert_array_equal(got, want)


def test_attention_with_sixteen_rows_per_group():
    """GQA ratio 16: every row of the 16-row tensor-core tile is a real query head."""
    wl = workloads.sink_local_fp32(seed=44, B=1, Hq=16, Hkv=1, S=1500, D=128, sink=8, window=40)
    rng = np.random.default_rng(11)
    for dtype in ("bf16", "f32"):
        q, k, v = (workloads.to_dtype(a, dtype) for a in (wl.q, wl.k, wl.v))
        dense = (rng.random((1, 16, 1, 1500)) < 0.2).astype(np.float32)
        dense[..., :8] = 1.0
        tq, tk, tv = (workloads.to_torch(a, dtype, DEV) for a in (q, k, v))
        m = Mask.create_mask_from_dense_mask(dense.shape, workloads.to_torch(dense, dtype, DEV),
                                             workloads.torch_dtype(dtype))
        out = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), m)
        ref = o_attention.masked_attention(q, k, v, dense, wl.scaling, dtype)
        _close(out.float().cpu().numpy(), ref, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gpu_mask_interop_from_rows_and_sparse_merge(dtype):
    """`Mask.create_from_row_wise_idx(mode="dense")` and `merge_mask(mode="sparse")` on device
    tensors run the library's scatter / flat-add kernels; both must give the reference's result
    bit for bit (duplicates inside a row: the last one stays; merged entries: summed in the mask
    dtype, clamped, every stored index kept)."""
    g = load_golden(f"mask_interop_{dtype}")
    td = workloads.torch_dtype(dtype)
    shape = tuple(g["row_dense"].shape)
    idx = torch.from_numpy(g["row_idx"]).to(DEV)
    vals = workloads.to_torch(g["row_vals"], dtype, DEV)
    m = Mask.create_from_row_wise_idx(shape, idx, vals, mask_type="dense", dtype=td, mode="dense")
    np.testing.assert_array_equal(m.get_dense_mask().float().cpu().numpy(), g["row_dense"])
    np.testing.assert_array_equal(m.get_dense_mask().float().cpu().numpy(),
                                  mask_ops.from_row_wise_idx(shape, g["row_idx"], g["row_vals"]))

    def index_form(dense):
        d = Mask.create_mask_from_dense_mask(shape, workloads.to_torch(dense, dtype, DEV), td)
        i, p, v = d.get_index_mask()
        return Mask.create_mask_from_indices(shape, i, p, v, td)

    merged = index_form(g["a"]).merge_mask(index_form(g["b"]), inplace=False, mode="sparse")
    mi, mp, md = merged.get_index_mask()
    np.testing.assert_array_equal(mi.cpu().numpy(), g["merged_idx"])
    np.testing.assert_array_equal(mp.cpu().numpy(), g["merged_ptr"])
    np.testing.assert_array_equal(md.float().cpu().numpy(), g["merged_data"])
    oi, op, od = mask_ops.merge_sparse(g["a"], g["b"], dtype)
    np.testing.assert_array_equal(mi.cpu().numpy(), oi)
    np.testing.assert_array_equal(md.float().cpu().numpy(), od)


@pytest.mark.gpu
@pytest.mark.parametrize("hidden,layers,bits,act", [(128, 3, 32, "silu"), (64, 2, 16, "relu"), (32, 3, 32, "gelu")])
def test_hash_signatures_from_tensor_cores_equal_the_fixed_order_kernel(hidden, layers, bits, act,
                                                                        monkeypatch):
    """On request (SAH_HASH_TC=1) ranges of 1024 keys and more are hashed with the layers'
    products on the tensor cores and every output near a bfloat16 rounding midpoint redone in the
    fixed order; shorter ranges take the fixed-order kernel.  Hashing 6000 keys in one call and in
    slices of 1000 must give the same words -- and those are the restatement's codes."""
    monkeypatch.setenv("SAH_HASH_TC", "1")
    S, B, Hkv, Hq, D = 6000, 2, 2, 4, 128
    w = workloads.hat_weights(31 + hidden, Hq, D, hidden, bits, layers)
    rng = np.random.default_rng(3)
    w["key_bias"] = [(rng.standard_normal(b.shape) * 0.1).astype(np.float32) for b in w["key_bias"]]
    k = workloads.to_dtype((rng.standard_normal((B, Hkv, S, D)) * 0.8).astype(np.float32), "bf16")
    tk = workloads.to_torch(k, "bf16", DEV)
    weights = [workloads.to_torch(a, "bf16", DEV).contiguous() for a in w["key_matrix"]]
    biases = [workloads.to_torch(a, "bf16", DEV).contiguous() for a in w["key_bias"]]
    whole = torch.zeros((B, Hq, S), dtype=torch.int32, device=DEV)
    sliced = torch.zeros_like(whole)
    _native_ops.hash_encode(tk, Hq, weights, biases, act, whole, 0, S)
    for s0 in range(0, S, 1000):
        _native_ops.hash_encode(tk, Hq, weights, biases, act, sliced, s0, min(S, s0 + 1000))
    torch.cuda.synchronize()
    assert torch.equal(whole, sliced)
    n = 256
    mats = [workloads.to_dtype(a, "bf16") for a in w["key_matrix"]]
    bias = [workloads.to_dtype(a, "bf16") for a in w["key_bias"]]
    ref = o_hash.signatures(o_attention.repeat_kv(k[:, :, :n], Hq // Hkv), mats, bias, act, "bf16")
    np.testing.assert_array_equal(whole[:, :, :n].cpu().numpy().view(np.uint32), ref)
