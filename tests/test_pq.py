"""PQCache: numpy restatement vs the reference's fixtures (CPU) and CUDA path vs both (GPU).

Integer results (codes, index sets) are compared bit for bit.  k-means is compared in lock
step: from the reference's own initial centres one Lloyd iteration must give the same
assignment and centres within 1e-5; after five iterations a handful of boundary keys may sit
in a different cluster because the reference sums cluster members in fp32 in its own order
(bounded below).  The decode step is compared on the reference-built codebook, where it must
reproduce the reference mask exactly.
"""

import numpy as np
import pytest

from oracle import mask_ops, pq, stacks
import workloads

from conftest import load_golden

N_SUB, CENT, OFF = 16, 16, 4


def _workload():
    return workloads.pqcache(seed=41, dtype="bf16", B=1, Hq=8, Hkv=2, S=600, D=128, sink=4,
                             window=16, heavy=32, group_factor=16, bits=4, kmeans_iter=5,
                             n_clusters=16)


def _check_mask(mask, g, prefix):
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g[prefix + "idx"])
    np.testing.assert_array_equal(ptr, g[prefix + "ptr"])
    np.testing.assert_array_equal(data, g[prefix + "data"])


# ------------------------------------------------------------------ CPU: oracle vs reference
def test_kmeans_lock_step_against_reference():
    g = load_golden("pq_kmeans_lockstep")
    wl = _workload()
    X = pq.split_keys(wl.k, OFF, N_SUB)
    init = X[np.arange(X.shape[0])[:, None], g["init_idx"]]
    reseed = [g["reseed"]] * 5  # the draws the reference was handed, one table per iteration
    codes1, cent1 = pq.kmeans(X, init, 1, reseed)
    np.testing.assert_array_equal(codes1, g["codes1"])
    # the reference returns centres cast to the key dtype
    np.testing.assert_allclose(workloads.to_dtype(cent1, "bf16"), g["centers1"], atol=1e-5, rtol=8e-3)
    codes5, cent5 = pq.kmeans(X, init, 5, reseed)
    assert np.mean(codes5 != g["codes5"]) < 5e-3
    np.testing.assert_allclose(workloads.to_dtype(cent5, "bf16"), g["centers5"], atol=2e-2, rtol=2e-2)


def test_pq_decode_exact_on_reference_codebook():
    g = load_golden("pq_stack_bf16")
    wl = _workload()
    n_first = 592 - OFF
    codes = g["codes_first"].transpose(0, 2, 1, 3)  # [B,n,Hkv,n_sub] -> [B,Hkv,n,n_sub]
    meta = {"pq_centroids": g["centroids"], "pq_codes": codes}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k[:, :, :592], wl.v[:, :, :592], wl.scaling,
                                    "bf16", meta=meta)
    assert codes.shape[2] == n_first
    _check_mask(mask, g, "first_")
    np.testing.assert_allclose(out, g["first_out"], atol=2e-2, rtol=2e-2)


def test_pq_appended_keys_quantised_like_reference():
    g = load_golden("pq_stack_bf16")
    wl = _workload()
    X_new = pq.split_keys(wl.k[:, :, 592:], 0, N_SUB)
    C = g["centroids"].reshape(-1, CENT, 8)
    new_codes = pq.assign(X_new, C, dtype_math="bf16").reshape(1, 2, N_SUB, 8).transpose(0, 1, 3, 2)
    want = g["codes_after_append"].transpose(0, 2, 1, 3)[:, :, 588:]
    np.testing.assert_array_equal(new_codes, want)
    meta = {"pq_centroids": g["centroids"],
            "pq_codes": g["codes_after_append"].transpose(0, 2, 1, 3)}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=meta)
    _check_mask(mask, g, "append_")
    np.testing.assert_allclose(out, g["append_out"], atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------ GPU: kernels vs oracle / reference
def _native_stack(wl, meta):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    dev = "cuda:0"
    ra = workloads.research_attention(wl.stack, wl.dtype, dev)
    q, k, v = (workloads.to_torch(a, wl.dtype, dev) for a in (wl.q, wl.k, wl.v))
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    idx, ptr, data = mask.get_index_mask()
    return (idx.cpu().numpy(), ptr.cpu().numpy(), data.float().cpu().numpy()), out.float().cpu().numpy()


@pytest.mark.gpu
def test_gpu_kmeans_build_matches_oracle_bit_for_bit():
    import torch

    wl = _workload()
    groups = 1 * 2 * N_SUB
    init_idx = workloads.pq_init_indices(43, groups, 600 - OFF, CENT)
    reseed = np.random.default_rng(43).integers(0, 600 - OFF, size=(5, groups, CENT)).astype(np.int64)
    meta = {"pq_init_indices": {0: torch.from_numpy(init_idx)},
            "pq_reseed_indices": {0: torch.from_numpy(reseed)}}
    (idx, ptr, data), out = _native_stack(wl, meta)
    ometa = {"pq_init_indices": init_idx, "pq_reseed_indices": reseed}
    ref_mask, ref_out, ometa = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=ometa)
    got_codes = meta["pq_codebook"][0].codes[:, :, : 600 - OFF].cpu().numpy()
    np.testing.assert_array_equal(got_codes, ometa["pq_codes"])
    np.testing.assert_array_equal(meta["pq_centroids"][0].float().cpu().numpy(), ometa["pq_centroids"])
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(idx, ri)
    np.testing.assert_array_equal(ptr, rp)
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_decode_and_append_on_reference_codebook():
    import torch

    g = load_golden("pq_stack_bf16")
    wl = _workload()
    dev = "cuda:0"
    meta = {"pq_centroids": {0: workloads.to_torch(g["centroids"], "bf16", dev)},
            "pq_codebook": {0: torch.from_numpy(g["codes_first"]).to(dev)},  # reference layout
            "pq_ip2l2_phi": {0: None}}
    short = workloads.DecodeWorkload(wl.name, wl.dtype, wl.q, wl.k[:, :, :592], wl.v[:, :, :592],
                                     wl.scaling, wl.stack)
    (idx, ptr, data), out = _native_stack(short, meta)
    np.testing.assert_array_equal(idx, g["first_idx"])
    np.testing.assert_array_equal(ptr, g["first_ptr"])
    np.testing.assert_allclose(out, g["first_out"], atol=2e-2, rtol=2e-2)
    # eight keys appended: quantised against the stored centroids, then the same stack
    (idx, ptr, data), out = _native_stack(wl, meta)
    codes = meta["pq_codebook"][0].to_reference_layout().cpu().numpy()
    np.testing.assert_array_equal(codes, g["codes_after_append"])
    np.testing.assert_array_equal(idx, g["append_idx"])
    np.testing.assert_array_equal(ptr, g["append_ptr"])
    np.testing.assert_allclose(out, g["append_out"], atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("n_cent,n_keys", [(256, 20000), (16, 3000), (48, 777)])
def test_gpu_assignment_on_tensor_cores_equals_the_fixed_order_kernel(n_cent, n_keys):
    """`sah_pq_assign_tc` (tcgen05 distance contraction, fixed-order argmin among the near-minimal
    centroids) writes the codes of `sah_pq_assign`, including ties (duplicated centroids and keys
    that sit exactly on centroids) -- and those are the restatement's codes."""
    import torch
    from sparse_attention_hub import _native

    lib = _native.load()
    dev = "cuda:0"
    B, Hkv, n_sub, sub_d, off = 2, 2, 16, 8, 5
    D, S = n_sub * sub_d, n_keys + off
    gen = torch.Generator(device=dev).manual_seed(n_cent)
    keys = (torch.randn((B, Hkv, S, D), generator=gen, device=dev) * 1.5).to(torch.bfloat16)
    groups = B * Hkv * n_sub
    cent = torch.randn((groups, n_cent, sub_d), generator=gen, device=dev) * 1.2
    cent[:, 3] = cent[:, 1]                       # a duplicated centroid: the lower index must win
    sub = keys[:, :, off:].reshape(B, Hkv, n_keys, n_sub, sub_d)
    cent.view(B, Hkv, n_sub, n_cent, sub_d)[:, :, :, 5] = sub[:, :, 7].float()   # a key on a centroid
    cent = cent.contiguous()
    cap = n_keys + 11
    want = torch.full((B, Hkv, cap, n_sub), 255, dtype=torch.uint8, device=dev)
    got = torch.full_like(want, 254)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    st = _native.stream_of(torch.device(dev))
    _native.check(lib.sah_pq_assign(keys.data_ptr(), _native.SAH_BF16, keys.stride(0), keys.stride(1), keys.stride(2),
                                    B, Hkv, off, S, off, n_sub, sub_d, n_cent, cent.data_ptr(), want.data_ptr(), cap,
                                    0, st), "sah_pq_assign")
    _native.check(lib.sah_pq_assign_tc(keys.data_ptr(), keys.stride(0), keys.stride(1), keys.stride(2), B, Hkv, off,
                                       S, off, n_sub, sub_d, n_cent, cent.data_ptr(), got.data_ptr(), cap,
                                       err.data_ptr(), 148, st), "sah_pq_assign_tc")
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(got[:, :, :n_keys], want[:, :, :n_keys])
    assert bool((got[:, :, n_keys:] == 254).all())
    # the restatement on a slice
    n = min(n_keys, 400)
    X = pq.split_keys(keys[:, :, : off + n].float().cpu().numpy(), off, n_sub)
    codes = pq.assign(X, cent.cpu().numpy()).reshape(B, Hkv, n_sub, n).transpose(0, 1, 3, 2)
    np.testing.assert_array_equal(got[:, :, :n].cpu().numpy(), codes)


# ------------------------------------------------------------------ metric "ip"
def _ip_workload():
    wl = workloads.pqcache(seed=45, dtype="bf16", B=1, Hq=8, Hkv=2, S=600, D=128, sink=4, window=16,
                           heavy=32, group_factor=N_SUB, bits=4, kmeans_iter=5, n_clusters=16)
    wl.stack[-1][1]["metric"] = "ip"
    return wl


def test_pq_ip_metric_restatement_equals_the_reference():
    """The inner-product metric (utils/pq_utils.py:585-640): augmented clustering, scores on the
    first sub_d centroid columns -- phi, centroids, codes, index sets and output of the reference."""
    g = load_golden("pq_stack_ip_bf16")
    wl = _ip_workload()
    meta = {"pq_init_indices": g["init_idx"],
            "pq_reseed_indices": np.broadcast_to(g["reseed"], (5,) + g["reseed"].shape)}
    mask, out, meta = stacks.run_stack(wl.stack, wl.q, wl.k[:, :, :592], wl.v[:, :, :592], wl.scaling, "bf16",
                                       meta=meta)
    np.testing.assert_array_equal(meta["pq_ip2l2_phi"].reshape(-1), g["phi"].reshape(-1))
    np.testing.assert_array_equal(meta["pq_centroids"], g["centroids"])
    np.testing.assert_array_equal(meta["pq_codes"].transpose(0, 2, 1, 3), g["codes_first"])
    _check_mask(mask, g, "first_")
    np.testing.assert_allclose(out, g["first_out"], atol=2e-2, rtol=2e-2)


def test_pq_two_batches_two_query_positions_against_the_reference():
    """Reference fixture with B = 2 and Sq = 2 (euclidean): centroids, codes, index sets and output
    of the restatement are the reference's."""
    g = load_golden("pq_stack_bf16_sq2")
    wl = workloads.pqcache(seed=47, dtype="bf16", B=2, Hq=4, Hkv=2, S=400, D=128, sink=4, window=16,
                           heavy=24, group_factor=N_SUB, bits=4, kmeans_iter=5, n_clusters=16, Sq=2)
    meta = {"pq_init_indices": g["init_idx"],
            "pq_reseed_indices": np.broadcast_to(g["reseed"], (5,) + g["reseed"].shape)}
    mask, out, meta = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=meta)
    np.testing.assert_array_equal(meta["pq_centroids"], g["centroids"])
    np.testing.assert_array_equal(meta["pq_codes"].transpose(0, 2, 1, 3), g["codes_first"])
    _check_mask(mask, g, "first_")
    np.testing.assert_allclose(out, g["first_out"], atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_ip_metric_build_decode_and_append_equal_the_reference():
    import torch

    g = load_golden("pq_stack_ip_bf16")
    wl = _ip_workload()
    reseed = np.broadcast_to(g["reseed"], (5,) + g["reseed"].shape).copy()
    meta = {"pq_init_indices": {0: torch.from_numpy(g["init_idx"])},
            "pq_reseed_indices": {0: torch.from_numpy(reseed)}}
    short = workloads.DecodeWorkload(wl.name, wl.dtype, wl.q, wl.k[:, :, :592], wl.v[:, :, :592],
                                     wl.scaling, wl.stack)
    (idx, ptr, data), out = _native_stack(short, meta)
    np.testing.assert_array_equal(meta["pq_ip2l2_phi"][0].float().cpu().numpy().reshape(-1), g["phi"].reshape(-1))
    np.testing.assert_array_equal(meta["pq_centroids"][0].float().cpu().numpy(), g["centroids"])
    np.testing.assert_array_equal(meta["pq_codebook"][0].to_reference_layout().cpu().numpy(), g["codes_first"])
    np.testing.assert_array_equal(idx, g["first_idx"])
    np.testing.assert_array_equal(ptr, g["first_ptr"])
    np.testing.assert_allclose(out, g["first_out"], atol=2e-2, rtol=2e-2)
    # eight appended keys: a zero column instead of the augmentation (pq_top_k.py:371-383)
    (idx, ptr, data), out = _native_stack(wl, meta)
    np.testing.assert_array_equal(meta["pq_codebook"][0].to_reference_layout().cpu().numpy(),
                                  g["codes_after_append"])
    np.testing.assert_array_equal(idx, g["append_idx"])
    np.testing.assert_array_equal(ptr, g["append_ptr"])
    np.testing.assert_allclose(out, g["append_out"], atol=2e-2, rtol=2e-2)
