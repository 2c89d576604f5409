"""OracleTopP: numpy restatement vs the reference's fixture (CPU) and the CUDA path vs both (GPU).

The selection hangs on a float32 running sum taken in sorted order and rounded to bfloat16
prefix by prefix; the restatement adds one value after the other like the reference does, the
kernel replays the same accumulator over runs of equal values.  Index sets are compared bit for
bit.  The fixture holds the reference's own q.k (torch.matmul); the restatement and the kernel
are pinned on those scores, and compared with each other on their shared q.k order.
"""

import numpy as np
import pytest

from oracle import mask_ops, stacks, topp
import workloads

from conftest import load_golden

CASES = (("p50", 0.5, False), ("p90", 0.9, False), ("p99", 0.99, False), ("masked", 0.9, True))


def _workload():
    return workloads.oracle_topk(seed=71, dtype="bf16", B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16, window=32)


def _stack(top_p):
    return [("sink", {"sink_size": 16}), ("local", {"window_size": 32}), ("oracle_topp", {"top_p": top_p})]


@pytest.mark.parametrize("tag,top_p,masked", CASES)
def test_restatement_against_reference(tag, top_p, masked):
    g = load_golden("oracle_topp_bf16")
    wl = _workload()
    am = g["attention_mask"] if masked else None
    mask, out, _ = stacks.run_stack(_stack(top_p), wl.q, wl.k, wl.v, wl.scaling, "bf16", attention_mask=am,
                                    meta={"oracle_scores_in": g["scores"]})
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g[f"{tag}_idx"])
    np.testing.assert_array_equal(ptr, g[f"{tag}_ptr"])
    np.testing.assert_array_equal(data, g[f"{tag}_data"])
    np.testing.assert_allclose(out, g[f"{tag}_out"], atol=2e-2, rtol=2e-2)


def test_numpy_cumsum_is_the_sequential_float32_sum():
    from oracle.bf16 import round_bf16
    rng = np.random.default_rng(1)
    for n in (1, 7, 1000, 40000):
        x = np.sort(round_bf16(rng.random(n).astype(np.float32) ** 6))[::-1]
        np.testing.assert_array_equal(topp.sequential_prefix_sums(x), topp.sequential_prefix_sums_loop(x))


def test_threshold_edge_cases():
    w = np.array([1.0, 0.5, 0.5, 0.25, 0.0, 0.0], np.float32)
    assert topp.threshold_row(w, 0.0) == np.float32(1.0)        # the first prefix already exceeds 0
    assert topp.threshold_row(w, 1.0) == np.float32(0.0)        # never exceeded: clamped to the last element
    assert topp.threshold_row(w[:4], 1.0) == np.float32(0.25)
    assert topp.threshold_row(w, 0.5) == np.float32(0.5)        # 1/2.25 = 0.444 <= 0.5 < 1.5/2.25


def test_config_and_rules_cpu():
    import torch
    from sparse_attention_hub.sparse_attention import (Mask, OracleTopPMasker, OracleTopPMaskerConfig,
                                                       ResearchAttentionConfig, SparseAttention)

    with pytest.raises(ValueError):
        OracleTopPMaskerConfig(top_p=1.5)
    with pytest.raises(ValueError):
        OracleTopPMasker.create_from_config(object())
    m = OracleTopPMasker.create_from_config(OracleTopPMaskerConfig(top_p=1.0))
    q, k = torch.zeros(1, 2, 1, 8), torch.zeros(1, 2, 16, 8)
    prev = Mask.create_empty_mask((1, 2, 1, 16), torch.float32, torch.device("cpu"))
    assert m.add_mask(k, q, k, None, 1.0, 0.0, {}, prev).is_full_mask()      # S <= int(1.0 * S)
    m = OracleTopPMasker.create_from_config(OracleTopPMaskerConfig(top_p=0.5))
    with pytest.raises(NotImplementedError):                                   # float32 rows
        m.add_mask(k, q, k, None, 1.0, 0.0, {}, prev)
    sa = SparseAttention.create_from_config(
        ResearchAttentionConfig(masker_configs=[OracleTopPMaskerConfig(top_p=0.9)]))
    assert type(sa.maskers[0]) is OracleTopPMasker


# ------------------------------------------------------------------ GPU
def _native_select(scores, am, scaling, prev_np, top_p, or_prev=True):
    import torch
    from sparse_attention_hub.sparse_attention import Mask, _native_ops

    dev = torch.device("cuda:0")
    shape = scores.shape
    s = workloads.to_torch(scores, "bf16", dev)
    prev = Mask.create_mask_from_dense_mask(shape, torch.from_numpy(prev_np.astype(np.float32)).to(dev).to(torch.bfloat16),
                                            torch.bfloat16)
    amt = None if am is None else workloads.to_torch(am, "bf16", dev)
    sel = _native_ops.topp_select(s, amt, scaling, prev, top_p, or_prev)
    return Mask._from_native(shape, torch.bfloat16, sel).get_dense_mask().float().cpu().numpy() != 0


@pytest.mark.gpu
@pytest.mark.parametrize("tag,top_p,masked", CASES)
def test_gpu_kernel_on_reference_scores(tag, top_p, masked):
    """The kernel, given the reference's q.k, reproduces the reference's index set."""
    g = load_golden("oracle_topp_bf16")
    wl = _workload()
    S = 1024
    prev = np.zeros(g["scores"].shape, bool)
    prev[..., :16] = True
    prev[..., S - 32:] = True
    am = g["attention_mask"] if masked else None
    got = _native_select(g["scores"], am, float(wl.scaling), prev, top_p)
    rows, cols = np.nonzero(got.reshape(-1, S))
    np.testing.assert_array_equal(rows * S + cols, g[f"{tag}_idx"])


@pytest.mark.gpu
@pytest.mark.parametrize("tag,top_p,masked", CASES)
def test_gpu_stack_against_restatement(tag, top_p, masked):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    g = load_golden("oracle_topp_bf16")
    wl = _workload()
    am = g["attention_mask"] if masked else None
    ref_mask, ref_out, _ = stacks.run_stack(_stack(top_p), wl.q, wl.k, wl.v, wl.scaling, "bf16", attention_mask=am)
    dev = "cuda:0"
    ra = workloads.research_attention(_stack(top_p), "bf16", dev)
    q, k, v = (workloads.to_torch(a, "bf16", dev) for a in (wl.q, wl.k, wl.v))
    amt = None if am is None else workloads.to_torch(am, "bf16", dev)
    mask = ra.build_mask(q, k, v, amt, float(wl.scaling), 0.0, {}, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, amt, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    idx, ptr, data = mask.get_index_mask()
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(idx.cpu().numpy(), ri)
    np.testing.assert_array_equal(ptr.cpu().numpy(), rp)
    np.testing.assert_array_equal(data.float().cpu().numpy(), rd)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref_out, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("S,levels,top_p", [(32768, 0, 0.9), (32768, 7, 0.95), (20000, 3, 0.5),
                                           (5000, 1, 0.99), (70000, 40, 0.999), (4099, 0, 1.0),
                                           (4099, 0, 0.0)])
def test_gpu_long_rows_and_runs_of_equal_weights(S, levels, top_p):
    """Rows long enough for the accumulator to cross many binades, and rows whose weights take
    only a few values (long runs of equal addends: the replay jumps through them)."""
    from oracle.bf16 import round_bf16

    rng = np.random.default_rng(S + levels)
    rows = 6
    if levels:
        vals = round_bf16(rng.normal(0.0, 30.0, levels).astype(np.float32))
        sc = vals[rng.integers(0, levels, (1, rows, 1, S))]
    else:
        sc = round_bf16(rng.normal(0.0, 25.0, (1, rows, 1, S)).astype(np.float32))
    sc = sc.astype(np.float32)
    prev = np.zeros(sc.shape, bool)
    prev[..., :9] = True
    prev[0, 1, 0, rng.integers(0, S, 500)] = True
    scaling = 0.08838834764831845
    want = topp.select(sc, scaling, None, prev, top_p) | prev
    got = _native_select(sc, None, scaling, prev, top_p)
    np.testing.assert_array_equal(got, want)
    only = _native_select(sc, None, scaling, prev, top_p, or_prev=False)
    np.testing.assert_array_equal(only, topp.select(sc, scaling, None, prev, top_p))


@pytest.mark.gpu
def test_gpu_weighted_previous_mask_merges_like_the_reference():
    """After a sampling masker the previous mask carries weights below 1: selected keys get
    weight 1 through the dense merge clamp(previous + 1, 0, 1)."""
    import torch
    wl = workloads.oracle_topk(seed=73, dtype="bf16", B=1, Hq=4, Hkv=2, S=2048, D=64, sink=8, window=16)
    stack = [("sink", {"sink_size": 8}), ("random_sampling", {"sampling_rate": 0.05}),
             ("oracle_topp", {"top_p": 0.8})]
    draws = np.random.default_rng(3).integers(0, 2048, (1, 4, 1, int(0.05 * 2048)))
    ref_mask, _, _ = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                      meta={"random_sampling_draws": draws})
    dev = "cuda:0"
    ra = workloads.research_attention(stack, "bf16", dev)
    q, k, v = (workloads.to_torch(a, "bf16", dev) for a in (wl.q, wl.k, wl.v))
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0,
                         {"random_sampling_draws": {0: torch.from_numpy(draws)}}, layer_idx=0)
    idx, ptr, data = mask.get_index_mask()
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(idx.cpu().numpy(), ri)
    np.testing.assert_array_equal(data.float().cpu().numpy(), rd)


def test_restatement_three_query_positions_under_a_causal_mask():
    """Reference fixture with three query positions under an HF causal mask (the additive mask
    joins the scores before the softmax weights are ranked): same index sets, weights, output."""
    g = load_golden("oracle_topp_bf16_sq3_causal")
    wl = workloads.oracle_topk(seed=72, dtype="bf16", B=2, Hq=4, Hkv=2, S=640, D=64, sink=8, window=24, Sq=3)
    stack = [("sink", {"sink_size": 8}), ("local", {"window_size": 24}), ("oracle_topp", {"top_p": 0.8})]
    mask, out, _ = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                    attention_mask=g["attention_mask"], meta={"oracle_scores_in": g["scores"]})
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])
    np.testing.assert_allclose(out, g["out"], atol=2e-2, rtol=2e-2)
