"""The numpy restatement (`oracle/`) against outputs of the reference itself.

The fixtures under tests/golden/ were produced by tests/golden/make_golden.py,
which runs skylight-org/sparse-attention-hub on the same seeded inputs.
Integer results (index sets, ptr, hash codes) must match exactly wherever the
reference's arithmetic is order-independent; where a float summation order
decides a bit, the test feeds the reference's own codes / scores downstream and
still demands exact selections, and bounds the upstream disagreement.
Tolerances: attention outputs 1e-4 (fp32) and 2e-2 (bf16), abs and rel.
"""

import numpy as np
import pytest

import oracle
from oracle import attention, hashattention, mask_ops, qk, stacks, topk
import workloads

from conftest import load_golden

TOL = {"f32": 1e-4, "bf16": 2e-2}


def _check_mask(mask, g):
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])


def _check_out(out, g, dtype):
    np.testing.assert_allclose(out, g["out"], atol=TOL[dtype], rtol=TOL[dtype])


def test_sink_local_f32():
    g = load_golden("sink_local_f32")
    wl = workloads.sink_local_fp32(seed=11, B=1, Hq=8, Hkv=2, S=640, D=128, sink=16, window=48)
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "f32")
    _check_mask(mask, g)
    _check_out(out, g, "f32")


def test_sink_local_sq3_causal_with_sink_logits():
    g = load_golden("sink_local_f32_sq3_causal_sinks")
    wl = workloads.sink_local_fp32(seed=12, B=2, Hq=4, Hkv=2, S=320, D=64, sink=8, window=24, Sq=3)
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "f32",
                                    attention_mask=g["attention_mask"], sinks=g["sinks"])
    _check_mask(mask, g)
    _check_out(out, g, "f32")


def test_sink_local_bf16_fraction_sizes():
    g = load_golden("sink_local_bf16_fraction")
    wl = workloads.sink_local_fp32(seed=13, B=2, Hq=8, Hkv=4, S=512, D=128)
    q, k, v = (workloads.to_dtype(a, "bf16") for a in (wl.q, wl.k, wl.v))
    stack = [("sink", {"sink_size": 0.05}), ("local", {"window_size": 0.1})]
    mask, out, _ = stacks.run_stack(stack, q, k, v, wl.scaling, "bf16")
    _check_mask(mask, g)
    _check_out(out, g, "bf16")


def test_hash_signatures_close_to_reference():
    """Sign bits agree with the reference except where the pre-sign activation is
    within accumulation-order noise of zero."""
    g = load_golden("hash_bf16")
    wl = workloads.hashattention_bf16(seed=21, B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16, window=32)
    prm = wl.stack[2][1]
    w = prm["weights"]
    y = hashattention.mlp_outputs(attention.repeat_kv(wl.k, 4), w["key_matrix"], w["key_bias"],
                                  "silu", "bf16")
    codes = hashattention.pack_signs(y)
    diff = codes ^ g["kcodes"]
    n_bad = int(np.bitwise_count(diff).sum())
    assert n_bad <= 2e-3 * codes.size * 32, n_bad
    # every disagreeing bit sits on an activation that is tiny next to the typical one
    bad_bits = ((diff[..., None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool)
    typical = np.median(np.abs(y))
    assert np.all(np.abs(y[bad_bits]) <= 0.05 * typical)
    yq = hashattention.mlp_outputs(wl.q, w["query_matrix"], w["query_bias"], "silu", "bf16")
    assert int(np.bitwise_count(hashattention.pack_signs(yq) ^ g["qcodes"]).sum()) <= 2
    assert int(g["zero_signs"]) == 0


def test_hash_stack_exact_given_reference_codes():
    g = load_golden("hash_bf16")
    wl = workloads.hashattention_bf16(seed=21, B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16, window=32)
    meta = {"hash_kcodes": g["kcodes"], "hash_qcodes_in": g["qcodes"]}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=meta)
    _check_mask(mask, g)
    _check_out(out, g, "bf16")


@pytest.mark.parametrize("dtype,seed", [("bf16", 31), ("f32", 32)])
def test_oracle_topk(dtype, seed):
    g = load_golden(f"oracle_topk_{dtype}")
    wl = workloads.oracle_topk(seed=seed, dtype=dtype, B=2, Hq=8, Hkv=2, S=1024, D=128, sink=16,
                               window=32, heavy=0.02)
    # (1) scores: same values up to summation order
    s = qk.qk_scores(wl.q, wl.k, dtype)
    if dtype == "bf16":
        ulp = np.abs(g["scores"]) * 2.0 ** -7 + 1e-30
        assert np.all(np.abs(s - g["scores"]) <= ulp)
        assert np.mean(s != g["scores"]) < 0.02
    else:
        np.testing.assert_allclose(s, g["scores"], rtol=1e-5, atol=1e-4)
    # (2) selection and output: exact given the reference's own scores
    meta = {"oracle_scores_in": g["scores"]}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=meta)
    _check_mask(mask, g)
    _check_out(out, g, dtype)
    # (3) end to end with the restatement's own scores: sets differ only at near-ties
    mask2, out2, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype)
    assert np.mean((mask2 != 0) != (mask != 0)) < 1e-3
    np.testing.assert_allclose(out2, g["out"], atol=TOL[dtype] * 2, rtol=TOL[dtype] * 2)


def test_topk_tie_rule_lowest_column():
    s = np.array([[1.0, 3.0, 3.0, 2.0, 3.0, 0.0, 3.0]], np.float32)
    prev = np.zeros_like(s, bool)
    prev[0, 1] = True
    sel = topk.topk_inactive(s, prev, 2)
    assert sel.tolist() == [[False, False, True, False, True, False, False]]
    assert topk.topk_inactive(s, prev, 10).sum() == 6  # fewer candidates than k: all of them


def test_inverse_weight_rounding():
    m = np.array([1.0, 0.5, 0.0, 0.05078125], np.float32)
    w32 = mask_ops.inv_weights(m, "f32")
    assert w32[0] == np.float32(1.0) / (np.float32(1.0) + np.float32(1e-6)) and w32[2] == 0
    wbf = mask_ops.inv_weights(m, "bf16")
    assert wbf[0] == 1.0 and wbf[1] == 2.0 and wbf[2] == 0.0


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mask_interop_restatements(dtype):
    """Row-wise construction (last duplicate wins) and the sparse merge (sum, clamp, union of
    the stored entries) against what the reference's Mask produced."""
    g = load_golden(f"mask_interop_{dtype}")
    shape = g["row_dense"].shape
    np.testing.assert_array_equal(mask_ops.from_row_wise_idx(shape, g["row_idx"], g["row_vals"]), g["row_dense"])
    idx, ptr, data = mask_ops.merge_sparse(g["a"], g["b"], dtype)
    np.testing.assert_array_equal(idx, g["merged_idx"])
    np.testing.assert_array_equal(ptr, g["merged_ptr"])
    np.testing.assert_array_equal(data, g["merged_data"])


@pytest.mark.parametrize("act,seed", [("relu", 22), ("gelu", 23), ("tanh", 24)])
def test_hash_other_activations_against_the_reference(act, seed):
    """The other activations of the reference's map, two-layer MLPs: sign bits agree with the
    reference's except where the pre-sign output is within accumulation-order noise of zero (relu
    leaves exact zeros, which the reference's sign() maps to 0 and the packing to a cleared bit,
    as here); selection and output are exact given the reference's codes."""
    g = load_golden(f"hash_bf16_{act}")
    wl = workloads.hashattention_bf16(seed=seed, B=1, Hq=4, Hkv=2, S=777, D=128, sink=4, window=9,
                                      heavy=40, bits=32, hidden=64, layers=2, activation=act)
    w = wl.stack[2][1]["weights"]
    y = hashattention.mlp_outputs(attention.repeat_kv(wl.k, 2), w["key_matrix"], w["key_bias"], act, "bf16")
    codes = hashattention.pack_signs(y)
    diff = codes ^ g["kcodes"]
    n_bad = int(np.bitwise_count(diff).sum())
    assert n_bad <= 2e-3 * codes.size * 32, n_bad
    bad_bits = ((diff[..., None] >> np.arange(32, dtype=np.uint32)) & 1).astype(bool)
    assert np.all(np.abs(y[bad_bits]) <= 0.05 * np.median(np.abs(y)))
    yq = hashattention.mlp_outputs(wl.q, w["query_matrix"], w["query_bias"], act, "bf16")
    assert int(np.bitwise_count(hashattention.pack_signs(yq) ^ g["qcodes"]).sum()) <= 2
    meta = {"hash_kcodes": g["kcodes"], "hash_qcodes_in": g["qcodes"]}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=meta)
    _check_mask(mask, g)
    _check_out(out, g, "bf16")


@pytest.mark.parametrize("dtype,seed", [("bf16", 33), ("f32", 34)])
def test_oracle_topk_three_query_positions_under_a_causal_mask(dtype, seed):
    """The additive attention mask joins the scores before the selection
    (oracle_top_k.py:70-76): from the reference's own score tensor the restatement reproduces
    the reference's mask and output for three query positions under an HF causal mask."""
    g = load_golden(f"oracle_topk_{dtype}_sq3_causal")
    wl = workloads.oracle_topk(seed=seed, dtype=dtype, B=2, Hq=4, Hkv=2, S=320, D=64, sink=8, window=24,
                               heavy=0.05, Sq=3)
    meta = {"oracle_scores_in": g["scores"]}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=meta,
                                    attention_mask=g["attention_mask"])
    _check_mask(mask, g)
    _check_out(out, g, dtype)


def test_hash_three_query_positions_under_a_causal_mask():
    """The additive attention mask joins the Hamming scores before the top-k
    (hashattention_top_k.py:343-371): from the reference's codes the restatement reproduces the
    reference's mask and output for three query positions under an HF causal mask."""
    g = load_golden("hash_bf16_sq3_causal")
    wl = workloads.hashattention_bf16(seed=25, B=2, Hq=4, Hkv=2, S=320, D=64, sink=8, window=24,
                                      heavy=0.1, bits=32, hidden=64, layers=3, activation="silu", Sq=3)
    w = wl.stack[2][1]["weights"]
    y = hashattention.mlp_outputs(attention.repeat_kv(wl.k, 2), w["key_matrix"], w["key_bias"], "silu", "bf16")
    assert int(np.bitwise_count(hashattention.pack_signs(y) ^ g["kcodes"]).sum()) <= 2e-3 * y.size
    meta = {"hash_kcodes": g["kcodes"], "hash_qcodes_in": g["qcodes"]}
    mask, out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16", meta=meta,
                                    attention_mask=g["attention_mask"])
    _check_mask(mask, g)
    _check_out(out, g, "bf16")
