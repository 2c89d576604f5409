"""Adaptive and random sampling maskers: numpy restatement vs the reference's fixtures (CPU)
and the CUDA path vs the restatement (GPU).

The reference draws with `torch.randint`; the fixtures were made with those draws handed in,
and both the restatement and the CUDA path accept the same draws, so index sets are compared
bit for bit.  The adaptive budget is a float pipeline ending in a truncation to integer: the
reference's `torch.std` and `sum` use their own summation order, so a row's budget may differ
from the reference's by a rounding step of the mask dtype (bounds below); between the
restatement and the CUDA kernels, which share one summation order, budgets are identical.
"""

import numpy as np
import pytest

from oracle import mask_ops, sampling, stacks
import workloads

from conftest import load_golden

ADAPTIVE = {"f32": 51, "bf16": 52}


def _adaptive_workload(dtype, eps):
    return workloads.oracle_adaptive(seed=ADAPTIVE[dtype], dtype=dtype, B=2, Hq=8, Hkv=2, S=1024,
                                     D=128, sink=16, window=32, heavy=0.02, base_rate=0.05,
                                     epsilon=eps, delta=0.05)


def test_philox_known_answers():
    # Philox4x32-10 test vectors of the Random123 distribution (counter, key -> first word)
    assert int(sampling.philox_u32(0, np.array([0], np.uint64))[0]) == 0x6627E8D5
    ones = (0xFFFFFFFF << 32) | 0xFFFFFFFF
    # counter (ffffffff, ffffffff, 0, 0) is not a published vector; check determinism and range
    a = sampling.draw_columns(7, np.arange(100000, dtype=np.uint64), 16, 976)
    assert a.min() >= 16 and a.max() < 16 + 976
    assert abs(a.mean() - (16 + 975 / 2)) < 3.0
    np.testing.assert_array_equal(a, sampling.draw_columns(7, np.arange(100000, dtype=np.uint64), 16, 976))
    assert sampling.philox_u32(ones, np.array([1], np.uint64)).dtype == np.uint32


def test_fixed_sum_matches_exact_sum():
    x = np.random.default_rng(0).random(5000).astype(np.float32)
    assert abs(float(sampling.fixed_sum(x)) - float(x.astype(np.float64).sum())) < 1e-2


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_adaptive_against_reference(dtype):
    g = load_golden(f"adaptive_{dtype}")
    wl = _adaptive_workload(dtype, float(g["epsilon"]))
    meta = {"oracle_scores_in": g["scores"], "oracle_scores_unbiased": g["scores"],
            "adaptive_base_draws": g["base"], "adaptive_pool": g["pool"]}
    mask, out, meta = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=meta)
    stats = meta["adaptive_stats"]
    tol = 1e-4 if dtype == "f32" else 1.6e-2  # two bf16 rounding steps
    np.testing.assert_allclose(stats[:, 1], g["std"], rtol=tol)
    np.testing.assert_allclose(stats[:, 2], g["est_den"], rtol=tol)
    rel = np.abs(meta["adaptive_budget"] - g["budget"]) / g["budget"]
    assert rel.max() <= (2e-3 if dtype == "f32" else 7e-2), rel
    if np.array_equal(meta["adaptive_budget"], g["budget"]):
        idx, ptr, data = mask_ops.to_csr(mask)
        np.testing.assert_array_equal(idx, g["idx"])
        np.testing.assert_array_equal(ptr, g["ptr"])
        np.testing.assert_array_equal(data, g["data"])
        np.testing.assert_allclose(out, g["out"], atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)


def test_adaptive_two_query_positions_against_reference():
    """Reference fixture with two query positions (draws per (batch, head, query)): statistics
    and budgets as close to the reference's as its own summation order allows, and, where the
    budgets are equal, the same sampled sets, weights and output."""
    g = load_golden("adaptive_f32_sq2")
    wl = workloads.oracle_adaptive(seed=56, dtype="f32", B=2, Hq=4, Hkv=2, S=640, D=64, sink=16, window=32,
                                   heavy=0.02, base_rate=0.05, epsilon=float(g["epsilon"]), delta=0.05, Sq=2)
    meta = {"oracle_scores_in": g["scores"], "oracle_scores_unbiased": g["scores"],
            "adaptive_base_draws": g["base"], "adaptive_pool": g["pool"]}
    mask, out, meta = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "f32", meta=meta)
    stats = meta["adaptive_stats"]
    np.testing.assert_allclose(stats[:, 1], g["std"], rtol=1e-4)
    np.testing.assert_allclose(stats[:, 2], g["est_den"], rtol=1e-4)
    rel = np.abs(meta["adaptive_budget"] - g["budget"]) / g["budget"]
    assert rel.max() <= 2e-3, rel
    assert np.array_equal(meta["adaptive_budget"], g["budget"])
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])
    np.testing.assert_allclose(out, g["out"], atol=1e-4, rtol=2e-2)


def test_adaptive_mask_exact_on_reference_budget():
    """With the reference's budgets the sampled set and its weights are the reference's."""
    for dtype in ("f32", "bf16"):
        g = load_golden(f"adaptive_{dtype}")
        wl = _adaptive_workload(dtype, float(g["epsilon"]))
        meta = {"oracle_scores_in": g["scores"], "oracle_scores_unbiased": g["scores"]}
        mask, _, _ = stacks.run_stack(wl.stack[:3], wl.q, wl.k, wl.v, wl.scaling, dtype, meta=meta)
        rows, S = 16, 1024
        dense = np.zeros((rows, S), np.float32)
        pos = 0
        for r in range(rows):
            dense[r, g["pool"][pos:pos + g["budget"][r]]] = g["prob"][r]
            pos += g["budget"][r]
        merged = mask_ops.merge(mask, dense.reshape(mask.shape), dtype)
        idx, ptr, data = mask_ops.to_csr(merged)
        np.testing.assert_array_equal(idx, g["idx"])
        np.testing.assert_array_equal(ptr, g["ptr"])
        np.testing.assert_array_equal(data, g["data"])


def test_random_sampling_against_reference():
    g = load_golden("random_sampling_f32")
    wl = workloads.sink_local_fp32(seed=53, B=2, Hq=4, Hkv=2, S=512, D=64, sink=8, window=8)
    stack = [("sink", {"sink_size": 8}), ("random_sampling", {"sampling_rate": float(g["rate"])})]
    mask, out, _ = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, "f32",
                                    meta={"random_sampling_draws": g["draws"]})
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])
    np.testing.assert_allclose(out, g["out"], atol=1e-4, rtol=1e-4)


# ------------------------------------------------------------------ GPU: kernels vs restatement
def _native_stack(wl, meta, stack=None):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    dev = "cuda:0"
    ra = workloads.research_attention(stack or wl.stack, wl.dtype, dev)
    q, k, v = (workloads.to_torch(a, wl.dtype, dev) for a in (wl.q, wl.k, wl.v))
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    idx, ptr, data = mask.get_index_mask()
    return (idx.cpu().numpy(), ptr.cpu().numpy(), data.float().cpu().numpy()), out.float().cpu().numpy()


def _same_mask(got, ref_mask):
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(got[1], rp)
    np.testing.assert_array_equal(got[0], ri)
    np.testing.assert_array_equal(got[2], rd)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_gpu_adaptive_with_reference_draws(dtype):
    import torch

    g = load_golden(f"adaptive_{dtype}")
    wl = _adaptive_workload(dtype, float(g["epsilon"]))
    # the pool is as long as the reference's total budget; keep spare draws in case a row differs
    pool = np.concatenate([g["pool"], g["pool"][::-1]])
    meta = {"adaptive_sampling_draws": {0: {"base": torch.from_numpy(g["base"]),
                                            "pool": torch.from_numpy(pool)}}}
    got, out = _native_stack(wl, meta)
    ometa = {"adaptive_base_draws": g["base"], "adaptive_pool": pool}
    ref_mask, ref_out, ometa = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=ometa)
    budget, prob, stats = meta["adaptive_sampling_stats"][0]
    np.testing.assert_array_equal(budget.cpu().numpy(), ometa["adaptive_budget"])
    np.testing.assert_array_equal(prob.float().cpu().numpy(), ometa["adaptive_prob"])
    np.testing.assert_array_equal(stats.cpu().numpy(), ometa["adaptive_stats"])
    _same_mask(got, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)
    # and the reference's own budgets, up to one rounding step of the dtype per row
    rel = np.abs(budget.cpu().numpy() - g["budget"]) / g["budget"]
    assert rel.max() <= (2e-3 if dtype == "f32" else 7e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,Sq", [("bf16", 1), ("f32", 2)])
def test_gpu_adaptive_philox_draws(dtype, Sq):
    wl = workloads.oracle_adaptive(seed=54, dtype=dtype, B=1, Hq=8, Hkv=4, S=2048 + 40, D=64, sink=8,
                                   window=24, heavy=0.02, base_rate=0.03, epsilon=0.1, delta=0.1, Sq=Sq)
    seed = 5
    meta = {"adaptive_sampling_seed": seed}
    got, out = _native_stack(wl, meta)
    ometa = {"adaptive_seed": seed * 1000003}  # layer 0, first call
    ref_mask, ref_out, ometa = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=ometa)
    budget = meta["adaptive_sampling_stats"][0][0].cpu().numpy()
    np.testing.assert_array_equal(budget, ometa["adaptive_budget"])
    assert len(set(budget.tolist())) > 1
    _same_mask(got, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)
    # a second call of the same layer draws a different sample
    got2, _ = _native_stack(wl, meta)
    assert not np.array_equal(got2[0], got[0])


@pytest.mark.gpu
def test_gpu_adaptive_alone_on_empty_mask():
    """No previous mask: the static denominator is the plain sum (mask_attention_utils.py:95-98)."""
    wl = workloads.oracle_adaptive(seed=55, dtype="bf16", B=1, Hq=4, Hkv=2, S=1500, D=64, sink=0,
                                   window=0, heavy=0.02, base_rate=16, epsilon=0.03, delta=0.1)
    stack = [("adaptive_sampling", dict(wl.stack[-1][1], init_offset=0.01, local_offset=0.02))]
    meta = {"adaptive_sampling_seed": 9}
    got, out = _native_stack(wl, meta, stack)
    ref_mask, ref_out, ometa = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                                meta={"adaptive_seed": 9 * 1000003})
    _same_mask(got, ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_random_sampling_with_reference_draws():
    import torch

    g = load_golden("random_sampling_f32")
    wl = workloads.sink_local_fp32(seed=53, B=2, Hq=4, Hkv=2, S=512, D=64, sink=8, window=8)
    stack = [("sink", {"sink_size": 8}), ("random_sampling", {"sampling_rate": float(g["rate"])})]
    meta = {"random_sampling_draws": {0: torch.from_numpy(g["draws"])}}
    got, out = _native_stack(wl, meta, stack)
    np.testing.assert_array_equal(got[0], g["idx"])
    np.testing.assert_array_equal(got[1], g["ptr"])
    np.testing.assert_array_equal(got[2], g["data"])
    np.testing.assert_allclose(out, g["out"], atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
def test_gpu_random_sampling_own_draws_statistics():
    wl = workloads.sink_local_fp32(seed=56, B=1, Hq=8, Hkv=2, S=4096, D=64, sink=8, window=8)
    stack = [("random_sampling", {"sampling_rate": 0.25})]
    got, _ = _native_stack(wl, {}, stack)
    per_row = np.diff(got[1])
    # 1024 draws with replacement from 4096: about 4096 * (1 - exp(-1/4)) = 906 distinct
    assert np.all(per_row <= 1024) and abs(per_row.mean() - 906) < 30
    assert np.all(got[2] == np.float32(0.25))
