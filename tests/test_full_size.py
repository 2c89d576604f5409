"""The CUDA path against the numpy restatement at the sizes of the benchmark configurations
(one batch element each, so that the numpy side stays within minutes), plus the plan kernels
of long rows called directly.

Index sets, integer codes and budgets must be bit-exact; outputs within 2e-2 (bf16).  Where
the restatement cannot redo a whole index in bounded time, the part it does redo is stated in
the test: key signatures on a seeded sample of keys (HashAttention) or of 32768-key chunks
(MagicPig at 1M keys); everything after the signatures is checked over the whole sequence.
"""

import ctypes
import os

import numpy as np
import pytest
import torch

import workloads
from oracle import attention as o_attention
from oracle import hashattention as o_hash
from oracle import magicpig as o_magicpig
from oracle import mask_ops, stacks
from sparse_attention_hub import _native
from sparse_attention_hub.sparse_attention import Mask
from sparse_attention_hub.sparse_attention.utils import mask_attention_utils as mau
from sparse_attention_hub.sparse_attention.utils.mask import words_per_row

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CHUNK = 32768


def _run(wl, meta):
    ra = workloads.research_attention(wl.stack, wl.dtype, DEV)
    q, k, v = (workloads.to_torch(a, wl.dtype, DEV) for a in (wl.q, wl.k, wl.v))
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = mau.get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    return mask, out.float().cpu().numpy()


def _same_index_sets(mask: Mask, ref_dense: np.ndarray, weights: bool = True):
    idx, ptr, data = mask.get_index_mask()
    ri, rp, rd = mask_ops.to_csr(ref_dense)
    np.testing.assert_array_equal(ptr.cpu().numpy(), rp)
    np.testing.assert_array_equal(idx.cpu().numpy(), ri)
    if weights:
        np.testing.assert_array_equal(data.float().cpu().numpy(), rd)


def _device_workload(name, seed, S, stack, n_clusters):
    """A DecodeWorkload of the benchmark's long-sequence generator (keys and values made on the
    device chunk by chunk, each chunk from its own seed), copied to the host for the restatement."""
    B, Hq, Hkv, D = 1, 32, 8, 128
    k, v = workloads.clustered_kv_range(seed, B, Hkv, 0, S, D, DEV, "bf16", n_clusters=n_clusters)
    q = workloads.to_dtype(workloads._rng(seed, 0).standard_normal((B, Hq, 1, D), dtype=np.float32), "bf16")
    return workloads.DecodeWorkload(name, "bf16", q, k.float().cpu().numpy(), v.float().cpu().numpy(),
                                    1.0 / np.sqrt(D), stack), k, v


# ---------------------------------------------------------------------------
def test_hashattention_32768_keys():
    """Sink(128) + Local(512) + HashAttention top-k 5 % at 32 768 keys, 32/8 heads.  The key
    signatures of a seeded sample of 256 keys per head are redone exactly; selection, union
    list and attention are compared over all keys on the signatures of the CUDA path."""
    wl = workloads.hashattention_bf16(seed=0, B=1)
    S = wl.k.shape[2]
    meta: dict = {}
    mask, out = _run(wl, meta)
    kc = meta["key"][0]
    codes = kc.codes[..., : kc.length].cpu().numpy().view(np.uint32)
    cols = np.sort(np.random.default_rng(0).choice(S, 256, replace=False))
    w = wl.stack[2][1]["weights"]
    want = o_hash.signatures(o_attention.repeat_kv(wl.k, 4)[:, :, cols], w["key_matrix"], w["key_bias"],
                             "silu", "bf16")
    np.testing.assert_array_equal(codes[:, :, cols], want)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                            meta={"hash_kcodes": codes})
    assert ref_mask.sum() == 32 * (128 + 512 + 1638)
    _same_index_sets(mask, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)


def test_oracle_topk_adaptive_65536_keys():
    """Sink(128) + Local(512) + oracle top-k 2 % + adaptive sampling (base 5 %, eps = delta =
    0.05) at 65 536 keys: scores, budgets, sampled sets (Philox draws from one seed on both
    sides) and weights bit for bit, output within tolerance."""
    stack = workloads.oracle_adaptive(seed=0, B=1, S=256).stack
    wl, _, _ = _device_workload("oracle_adaptive_bf16", 3, 65536, stack, 64)
    seed = 11
    meta = {"adaptive_sampling_seed": seed}
    mask, out = _run(wl, meta)
    ref_mask, ref_out, ometa = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                                meta={"adaptive_seed": seed * 1000003})
    budget = meta["adaptive_sampling_stats"][0][0].cpu().numpy()
    np.testing.assert_array_equal(budget, ometa["adaptive_budget"])
    assert budget.min() >= 3244 and budget.max() <= 64896
    _same_index_sets(mask, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)


def test_pqcache_131072_keys():
    """Sink(64) + Local(256) + PQCache (16 sub-spaces x 256 centroids, 10 Lloyd iterations,
    top-2048) at 131 072 keys.  The codebook the CUDA path built is handed to the restatement
    (k-means in lock step is checked at a size the restatement can iterate); table scores,
    the 2048 selected keys per head and the output are compared over all keys."""
    stack = workloads.pqcache(seed=0, S=4096).stack
    wl, _, _ = _device_workload("pqcache_bf16", 4, 131072, stack, 256)
    meta: dict = {}
    mask, out = _run(wl, meta)
    n = 131072 - 64
    codes = meta["pq_codebook"][0].codes[:, :, :n].cpu().numpy()
    cent = meta["pq_centroids"][0].float().cpu().numpy()
    assert len(np.unique(codes)) == 256
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                            meta={"pq_centroids": cent, "pq_codes": codes})
    assert ref_mask.sum() == 32 * (64 + 256 + 2048)
    _same_index_sets(mask, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------------------
def _unpack(bits: torch.Tensor, S: int) -> np.ndarray:
    """uint32 bitmap words [rows, W] -> bool [rows, S]."""
    words = bits.cpu().numpy().view(np.uint32)
    return np.unpackbits(words.view(np.uint8), axis=-1, bitorder="little")[:, :S].astype(bool)


def _magicpig_against_chunked_oracle(S, sampled, seed, sharded_world=0):
    """MagicPig stack at S keys against `oracle.magicpig.chunked_step`.  The chunks in `sampled`
    have their key signatures redone by the restatement (index sets and weights compared bit
    for bit there); the other chunks take the CUDA path's matches and redo the probabilities,
    the merge with the sink / window bands and the attention partial.  Key mean, largest key
    norm and the merged output are over the whole sequence."""
    import bench

    stack = bench.long_stack("magicpig", seed, 32, 128)
    B, Hq, Hkv, D = 1, 32, 8, 128
    k_dev, v_dev = workloads.clustered_kv_range(seed, B, Hkv, 0, S, D, DEV, "bf16")
    q_np = workloads.to_dtype(workloads._rng(seed, 0).standard_normal((B, Hq, 1, D), dtype=np.float32), "bf16")
    wl = workloads.DecodeWorkload("magicpig_bf16", "bf16", q_np, None, None, 1.0 / np.sqrt(D), stack)
    proj = stack[-1][1]["projection"]
    ra = workloads.research_attention(stack, "bf16", DEV)
    q = workloads.to_torch(wl.q, "bf16", DEV)
    meta = {"projections": {0: workloads.to_torch(proj, "bf16", DEV)}}
    scaling = float(1.0 / np.sqrt(D))
    mask = ra.build_mask(q, k_dev, v_dev, None, scaling, 0.0, meta, layer_idx=0)
    payload = mask._native.deferred
    assert payload is not None, "bf16 decode must leave the weights to the attention kernel"
    out = mau.get_masked_attention_output(None, q, k_dev, v_dev, None, None, scaling, 0.0, mask)
    torch.cuda.synchronize()
    out = out.float().cpu().numpy()
    match = _unpack(payload.match_bits, S).reshape(B, Hq, 1, S)
    dense = mask.get_dense_mask().float().cpu().numpy()  # exact weights (probability kernel)

    def get_chunk(c0, c1):
        return (k_dev[:, :, c0:c1].float().cpu().numpy(), v_dev[:, :, c0:c1].float().cpu().numpy())

    checked = []

    def on_chunk(c0, c1, ref, codes):
        if codes is None:
            return
        np.testing.assert_array_equal(dense[..., c0:c1] != 0, ref != 0, err_msg=f"index set, keys {c0}:{c1}")
        np.testing.assert_array_equal(dense[..., c0:c1], ref, err_msg=f"weights, keys {c0}:{c1}")
        got = meta["key_signature"][0].codes[:, :, c0:c1, :75].cpu().numpy()
        np.testing.assert_array_equal(got.astype(np.int64), codes, err_msg=f"key codes, keys {c0}:{c1}")
        checked.append(c0)

    def known_match(c0, c1):
        return None if c0 // CHUNK in sampled else match[..., c0:c1]

    ref_out, st = o_magicpig.chunked_step(stack[-1][1], 64, 256, wl.q, get_chunk, S, CHUNK, "bf16", proj,
                                          scaling, on_chunk, known_match)
    assert len(checked) == len(sampled)
    np.testing.assert_array_equal(meta["key_mean"][0][:, ::4, 0, :].float().cpu().numpy(), st["mean"])
    M = meta["key_signature"][0].max_norm.cpu().numpy().view(np.float32)[0]
    assert M == st["M"]
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)
    density = (dense != 0).mean()
    assert 0.05 < density < 0.9
    return wl, k_dev, v_dev, stack, out, dense, ref_out


def test_magicpig_1048576_keys_chunked_oracle():
    """The 1M-key configuration on one GPU.  Chunks 0 (sink), 31 (window) and two seeded ones in
    between are redone in full; SAH_FULL_ORACLE=1 redoes all 32."""
    n = 1048576 // CHUNK
    if os.environ.get("SAH_FULL_ORACLE"):
        sampled = set(range(n))
    else:
        sampled = {0, n - 1} | set(np.random.default_rng(5).choice(np.arange(1, n - 1), 2, replace=False).tolist())
    _magicpig_against_chunked_oracle(1048576, sampled, seed=0)


def test_magicpig_65536_keys_two_ranks():
    """Two ranks (threads of this process, one device) over 65 536 keys: the union of the ranks'
    masks equals the unsharded mask and the restatement's, and every rank returns the merged
    output."""
    from test_sharded import _native_sharded, _proj_meta

    S = 65536
    wl, k_dev, v_dev, stack, out, dense, ref_out = _magicpig_against_chunked_oracle(S, {1}, seed=2)
    wl = workloads.DecodeWorkload("magicpig_bf16", "bf16", wl.q, k_dev.float().cpu().numpy(),
                                  v_dev.float().cpu().numpy(), wl.scaling, stack)
    plan, results = _native_sharded(wl, 2, _proj_meta(wl))
    union = np.concatenate([results[r][0] for r in range(2)], axis=-1)
    np.testing.assert_array_equal(union, dense)
    for r in range(2):
        np.testing.assert_allclose(results[r][1], out, atol=2e-2, rtol=2e-2)
        np.testing.assert_allclose(results[r][1], ref_out, atol=2e-2, rtol=2e-2)


def test_magicpig_in_kernel_weights_against_reference_fixture():
    """The weights the attention kernel evaluates in place, read back through its test hook,
    against the reference's own (tests/golden/magicpig_bf16.npz): the same entries, weights
    equal for most of them and within one bf16 step of the cosine for the rest (the kernel
    evaluates the cosine in float32 and rounds once; the reference rounds every step)."""
    from conftest import load_golden

    g = load_golden("magicpig_bf16")
    wl = workloads.magicpig(seed=61, dtype="bf16", B=1, Hq=8, Hkv=2, S=1024, D=128, sink=4, window=8,
                            lsh_l=75, lsh_k=8, n_clusters=8)
    ra = workloads.research_attention(wl.stack, "bf16", DEV)
    q, k, v = (workloads.to_torch(a, "bf16", DEV) for a in (wl.q, wl.k, wl.v))
    meta = {"projections": {0: workloads.to_torch(wl.stack[-1][1]["projection"], "bf16", DEV)}}
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    mau._weight_dump["request"] = True
    try:
        out = mau.native_masked_attention(q, k, v, None, None, float(wl.scaling), mask)
        torch.cuda.synchronize()
    finally:
        mau._weight_dump["request"] = None
    ucols, umemb, ucount, R = mau.last_union_list()
    S = 1024
    wts = mau._weight_dump["weights"].cpu().numpy().reshape(ucols.shape[0], S, R)
    ucols, umemb, ucount = ucols.cpu().numpy(), umemb.cpu().numpy().view(np.uint16), ucount.cpu().numpy()
    got = np.zeros((8, S), np.float32)        # inverse weights by (row, column)
    for g_ in range(ucols.shape[0]):
        for u in range(int(ucount[g_])):
            for r in range(R):
                if (umemb[g_, u] >> r) & 1:
                    got[g_ * R + r, ucols[g_, u]] = wts[g_, u, r]
    ref_dense = np.zeros((8, S), np.float32)
    rows = np.repeat(np.arange(8), np.diff(g["ptr"]))
    ref_dense[rows, g["idx"] - rows * S] = g["data"]
    want = mask_ops.inv_weights(ref_dense, "bf16")
    np.testing.assert_array_equal(got != 0, want != 0)
    sel = want != 0
    assert np.mean(got[sel] == want[sel]) > 0.6
    np.testing.assert_allclose(got[sel], want[sel], rtol=3.2e-2)
    np.testing.assert_allclose(out.float().cpu().numpy(), g["out"], atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------------------
def _plan_reference(bits_bool, weights, R, dtype):
    """numpy union list of groups of R consecutive rows: (ucols, umemb, uw, ucount) per group."""
    rows, S = bits_bool.shape
    out = []
    for g in range(rows // R):
        blk = bits_bool[g * R:(g + 1) * R]
        cols = np.flatnonzero(blk.any(axis=0))
        memb = (blk[:, cols].astype(np.uint16) << np.arange(R, dtype=np.uint16)[:, None]).sum(axis=0)
        uw = None
        if weights is not None:
            inv = mask_ops.inv_weights(weights[g * R:(g + 1) * R], dtype)
            uw = inv[:, cols].T.copy()
        out.append((cols.astype(np.int32), memb.astype(np.uint16), uw, cols.size))
    return out


@pytest.mark.parametrize("S,pad_words,with_data", [
    (70000, 0, False),    # count + emit kernels (rows longer than 32768 keys)
    (70000, 0, True),
    (300001, 12, False),  # ragged tail, row stride padded beyond ceil(S / 32)
    (20000, 0, False),    # one launch, three CTAs per group (blockIdx.y > 0)
    (20000, 8, True),
    (9000, 0, True),      # one launch, two CTAs per group, weights
])
def test_attn_plan_against_numpy_union(S, pad_words, with_data):
    """`sah_attn_plan` through the C ABI against a numpy union of the rows' bitmaps: ascending
    columns, membership, inverse weights, counts.  Words past ceil(S / 32) hold garbage and the
    last word has bits set beyond S: both must be ignored."""
    lib = _native.load()
    B, Hq, Hkv, Sq, D = 1, 8, 2, 1, 128
    rows, R = B * Hq * Sq, 4
    rng = np.random.default_rng(S + pad_words)
    dense = rng.random((rows, S)) < np.array([0.02, 0.3, 0.0, 0.7, 0.1, 0.1, 0.5, 0.01])[:, None]
    dense[:, :37] = True
    dense[1, S - 300:] = True
    W = words_per_row(S) + pad_words
    packed = np.zeros((rows, W * 32), bool)
    packed[:, :S] = dense
    packed[:, S:] = rng.random((rows, W * 32 - S)) < 0.5    # tail bits and padding words: garbage
    words = np.packbits(packed.reshape(rows, W, 32), axis=-1, bitorder="little").view(np.uint32).reshape(rows, W)
    bits = torch.from_numpy(words.view(np.int32)).to(DEV)
    dtype, tdt = "bf16", torch.bfloat16
    weights = data = wpre = ptr = None
    if with_data:
        weights = np.where(dense, workloads.to_dtype(rng.random((rows, S)).astype(np.float32) * 0.9 + 0.05, dtype), 0.0)
        # CSR companions of the caller's words as they are (garbage tail included), as the
        # row-scan kernel makes them
        pop = np.unpackbits(words.view(np.uint8), axis=-1, bitorder="little").reshape(rows, W, 32).sum(-1)
        wpre_np = np.cumsum(pop, axis=1) - pop
        ptr_np = np.concatenate([[0], np.cumsum(pop.sum(axis=1))]).astype(np.int64)
        flat = np.zeros(int(ptr_np[-1]), np.float32)
        for r in range(rows):
            cols = np.flatnonzero(packed[r])
            flat[ptr_np[r]:ptr_np[r + 1]] = np.where(cols < S, weights[r, np.minimum(cols, S - 1)], 0.5)
        data = workloads.to_torch(flat, dtype, DEV)
        wpre = torch.from_numpy(wpre_np.astype(np.int32)).to(DEV)
        ptr = torch.from_numpy(ptr_np).to(DEV)
    sizes = _native.AttnSizes()
    _native.check(lib.sah_attn_query_sizes(B, Hq, Hkv, Sq, S, D, int(with_data), 148, ctypes.byref(sizes)),
                  "sah_attn_query_sizes")
    ucols = torch.full((sizes.ucols_bytes // 4,), -7, dtype=torch.int32, device=DEV)
    umemb = torch.zeros(sizes.umemb_bytes // 2, dtype=torch.int16, device=DEV)
    uw = torch.zeros(max(1, sizes.uw_bytes // 4), dtype=torch.float32, device=DEV)
    ucount = torch.zeros(sizes.ucount_bytes // 4, dtype=torch.int32, device=DEV)
    _native.check(
        lib.sah_attn_plan(bits.data_ptr(), _native.ptr(data), _native.ptr(wpre), _native.ptr(ptr),
                          _native.SAH_BF16, B, Hq, Hkv, Sq, S, W, ctypes.byref(sizes), ucols.data_ptr(),
                          umemb.data_ptr(), uw.data_ptr() if with_data else None, ucount.data_ptr(),
                          _native.stream_of(torch.device(DEV))), "sah_attn_plan")
    torch.cuda.synchronize()
    groups = sizes.groups
    assert groups == 2 and sizes.rows_per_group == R
    # the merge tickets and the error word behind the counters stay zero
    nchunks = (words_per_row(S) + 31) // 32
    assert not ucount[groups + groups * nchunks:].any()
    uc, um = ucols.cpu().numpy().reshape(groups, S), umemb.cpu().numpy().view(np.uint16).reshape(groups, S)
    uwn = uw.cpu().numpy()
    for g, (cols, memb, w_ref, n) in enumerate(_plan_reference(dense, weights, R, dtype)):
        assert int(ucount[g]) == n
        np.testing.assert_array_equal(uc[g, :n], cols)
        np.testing.assert_array_equal(um[g, :n], memb)
        if with_data:
            got = uwn[g * S * R:(g * S + n) * R].reshape(n, R)
            np.testing.assert_array_equal(got, w_ref)
