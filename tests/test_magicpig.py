"""MagicPig: numpy restatement vs the reference's fixtures (CPU), CUDA path vs both (GPU).

Signature bits are signs of 129-term float sums; where a sum is within rounding of zero the
reference's BLAS order and the restatement's fixed order can disagree, so key codes are
compared as a mismatch count with a small bound, and everything downstream is checked on the
reference's own codes, where the sampled index set must be the reference's exactly.  The
weights are a chain of dtype-rounded operations on a 129-term dot product; they may differ
from the reference by one rounding step of the dtype (bound below).  Between the restatement
and the CUDA kernels, which share every order of operations, codes, index sets and weights
are identical.
"""

import numpy as np
import pytest

from oracle import magicpig, mask_ops, stacks
import workloads

from conftest import load_golden

CASES = {"magicpig_bf16": ("bf16", 61, 75, 8, 1024), "magicpig_f32": ("f32", 62, 12, 4, 512)}


def _workload(name):
    dtype, seed, L, K, S = CASES[name]
    return workloads.magicpig(seed=seed, dtype=dtype, B=1, Hq=8, Hkv=2, S=S, D=128, sink=4, window=8,
                              lsh_l=L, lsh_k=K, n_clusters=8)


def _oracle(wl, meta):
    meta = dict(meta)
    meta["lsh_projection"] = wl.stack[-1][1]["projection"]
    return stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, wl.dtype, meta=meta)


def test_bit_packing_order():
    # bit j of table l is column l*K + j (magic_pig.py:120-150)
    signs = np.zeros((1, 8), bool)
    signs[0, [0, 3, 5]] = True  # table 0: bits 0 and 3 -> 9; table 1: bit 1 -> 2
    np.testing.assert_array_equal(magicpig.pack(signs, 2, 4), [[9, 2]])


def test_probability_end_points():
    for dtype in ("f32", "bf16"):
        p = magicpig.collision_prob(np.array([1.0, -1.0, 0.0], np.float32), 4, 8, dtype)
        assert p[0] == 1.0 and p[1] == 0.0
        assert abs(p[2] - (1 - (1 - 0.5 ** 4) ** 8)) < 2e-2


@pytest.mark.parametrize("name", list(CASES))
def test_codes_against_reference(name):
    g = load_golden(name)
    wl = _workload(name)
    _, _, meta = _oracle(wl, {"lsh_key_mean": g["key_mean"]})
    kdiff = np.mean(meta["lsh_key_codes"] != g["key_sig"])
    qdiff = np.mean(meta["lsh_query_codes"] != g["query_sig"])
    assert kdiff < 2e-3 and qdiff < 2e-2, (kdiff, qdiff)


@pytest.mark.parametrize("name", list(CASES))
def test_mask_exact_on_reference_codes(name):
    g = load_golden(name)
    wl = _workload(name)
    dtype = CASES[name][0]
    state = {"codes": g["key_sig"].astype(np.int64), "norms": np.zeros((1, 2, 0), np.float32),
             "M": np.float32(0)}
    mask, out, _ = _oracle(wl, {"lsh_key_mean": g["key_mean"], "lsh_state": state,
                                "lsh_query_codes_in": g["query_sig"]})
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(idx, g["idx"])
    tol = 1.6e-2 if dtype == "bf16" else 1e-5
    np.testing.assert_allclose(data, g["data"], rtol=tol, atol=tol * 1e-2)
    assert np.mean(data != g["data"]) < (0.2 if dtype == "bf16" else 1.0)
    np.testing.assert_allclose(out, g["out"], atol=2e-2 if dtype == "bf16" else 1e-4, rtol=2e-2)


def test_two_query_positions_two_batches_against_reference():
    """The restatement on a reference fixture with B = 2, Sq = 2 and groups of two heads (the
    local window of a query position ends at its own key): codes close to the reference's,
    and index sets, weights and output from the reference's codes as the reference has them."""
    g = load_golden("magicpig_bf16_sq2")
    wl = workloads.magicpig(seed=64, dtype="bf16", B=2, Hq=4, Hkv=2, S=512, D=128, sink=4, window=8,
                            lsh_l=20, lsh_k=8, n_clusters=8, Sq=2)
    _, _, meta = _oracle(wl, {"lsh_key_mean": g["key_mean"]})
    assert np.mean(meta["lsh_key_codes"] != g["key_sig"]) < 2e-3
    assert np.mean(meta["lsh_query_codes"] != g["query_sig"]) < 2e-2
    state = {"codes": g["key_sig"].astype(np.int64), "norms": np.zeros((2, 2, 0), np.float32),
             "M": np.float32(0)}
    mask, out, _ = _oracle(wl, {"lsh_key_mean": g["key_mean"], "lsh_state": state,
                                "lsh_query_codes_in": g["query_sig"]})
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_allclose(data, g["data"], rtol=1.6e-2, atol=1.6e-4)
    np.testing.assert_allclose(out, g["out"], atol=2e-2, rtol=2e-2)


# ------------------------------------------------------------------ GPU: kernels vs restatement / reference
def _native_stack(wl, meta, k=None, v=None):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    dev = "cuda:0"
    ra = workloads.research_attention(wl.stack, wl.dtype, dev)
    q = workloads.to_torch(wl.q, wl.dtype, dev)
    k = workloads.to_torch(wl.k if k is None else k, wl.dtype, dev)
    v = workloads.to_torch(wl.v if v is None else v, wl.dtype, dev)
    meta.setdefault("projections", {})[0] = workloads.to_torch(wl.stack[-1][1]["projection"], wl.dtype, dev)
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    idx, ptr, data = mask.get_index_mask()
    return (idx.cpu().numpy(), ptr.cpu().numpy(), data.float().cpu().numpy()), out.float().cpu().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_gpu_magicpig_matches_oracle_and_reference(name):
    g = load_golden(name)
    wl = _workload(name)
    dtype = CASES[name][0]
    meta: dict = {}
    (idx, ptr, data), out = _native_stack(wl, meta)
    ref_mask, ref_out, ometa = _oracle(wl, {})
    # key mean, key codes
    mean = meta["key_mean"][0][:, ::4, 0, :].float().cpu().numpy()
    np.testing.assert_array_equal(mean, ometa["lsh_key_mean"])
    np.testing.assert_array_equal(mean, g["key_mean"])
    codes = meta["key_signature"][0].to_reference_layout(8)[:, ::4].cpu().numpy()
    np.testing.assert_array_equal(codes, ometa["lsh_key_codes"])
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(ptr, rp)
    np.testing.assert_array_equal(idx, ri)
    np.testing.assert_array_equal(data, rd)
    np.testing.assert_allclose(out, ref_out, atol=2e-2 if dtype == "bf16" else 1e-4, rtol=2e-2)
    # the reference itself
    np.testing.assert_array_equal(codes, g["key_sig"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(idx, g["idx"])
    tol = 1.6e-2 if dtype == "bf16" else 1e-5
    np.testing.assert_allclose(data, g["data"], rtol=tol, atol=tol * 1e-2)
    np.testing.assert_allclose(out, g["out"], atol=2e-2 if dtype == "bf16" else 1e-4, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_magicpig_adopts_reference_signature_cache():
    """A signature tensor cached by the reference (int64 [B,Hq,S,L]) is used as it is."""
    import torch

    name = "magicpig_bf16"
    g = load_golden(name)
    wl = _workload(name)
    sig = torch.from_numpy(np.repeat(g["key_sig"].astype(np.int64), 4, axis=1)).to("cuda:0")
    meta = {"key_signature": {0: sig},
            "key_mean": {0: workloads.to_torch(np.repeat(g["key_mean"], 4, axis=1)[:, :, None, :], "bf16", "cuda:0")}}
    (idx, ptr, data), out = _native_stack(wl, meta)
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(idx, g["idx"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,K,L,Sq", [("bf16", 8, 20, 1), ("f32", 10, 16, 2), ("bf16", 4, 6, 3)])
def test_gpu_magicpig_appended_keys(dtype, K, L, Sq):
    """Keys arriving after the first call are hashed with the maximum norm known then."""
    wl = workloads.magicpig(seed=63, dtype=dtype, B=2, Hq=4, Hkv=2, S=700, D=64, sink=4, window=8,
                            lsh_l=L, lsh_k=K, Sq=Sq, n_clusters=4)
    wl.k[:, :, 690:] *= 1.5  # larger norms among the appended keys move the maximum
    wl.k = workloads.to_dtype(wl.k, dtype)
    meta: dict = {}
    _native_stack(wl, meta, k=wl.k[:, :, :690], v=wl.v[:, :, :690])
    (idx, ptr, data), out = _native_stack(wl, meta)
    ometa = {"lsh_projection": wl.stack[-1][1]["projection"]}
    stacks.run_stack(wl.stack, wl.q, wl.k[:, :, :690], wl.v[:, :, :690], wl.scaling, dtype, meta=ometa)
    for key in ("lsh_key_codes", "lsh_query_codes", "lsh_match", "lsh_dense", "full", "empty"):
        ometa.pop(key, None)
    ref_mask, ref_out, ometa = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=ometa)
    codes = meta["key_signature"][0].to_reference_layout(4)[:, ::2].cpu().numpy()
    np.testing.assert_array_equal(codes, ometa["lsh_key_codes"])
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(ptr, rp)
    np.testing.assert_array_equal(idx, ri)
    np.testing.assert_array_equal(data, rd)
    np.testing.assert_allclose(out, ref_out, atol=2e-2 if dtype == "bf16" else 1e-4, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_merge_of_two_weighted_masks():
    """clamp(a + b, 0, 1) on bitmaps equals the dense merge (utils/mask.py:875-877)."""
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask import Mask

    rng = np.random.default_rng(5)
    shape = (2, 3, 2, 200)
    for dtype in (torch.float32, torch.bfloat16):
        a = torch.from_numpy((rng.random(shape) * (rng.random(shape) < 0.2)).astype(np.float32)).to("cuda:0", dtype)
        b = torch.from_numpy((rng.random(shape) * (rng.random(shape) < 0.3)).astype(np.float32)).to("cuda:0", dtype)
        ones = (torch.from_numpy(rng.random(shape) < 0.1).to("cuda:0")).to(dtype)
        for x, y in ((a, b), (a, ones), (ones, b)):
            ma = Mask.create_mask_from_dense_mask(shape, x, dtype)
            mb = Mask.create_mask_from_dense_mask(shape, y, dtype)
            na = Mask._from_native(shape, dtype, ma.native_bits())
            nb = Mask._from_native(shape, dtype, mb.native_bits())
            merged = na.merge_mask(nb, inplace=False)
            want = torch.clamp(x + y, 0.0, 1.0)
            assert torch.equal(merged.get_dense_mask(), want)


# ------------------------------------------------------------------ CPU: the restatement's own shortcuts
def test_fast_projection_signs_equal_the_fixed_order():
    """BLAS product + recomputation of the sums near zero gives the signs of the fixed order."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3000, 129)).astype(np.float32)
    p = rng.standard_normal((129, 64)).astype(np.float32)
    x[:50] = 0.0                                  # exact zeros: "not positive"
    x[50:200, 64:] = -x[50:200, :65][:, ::-1]     # sums that cancel almost exactly
    p[:64, :8] = p[64:128, :8][::-1]
    x[200] = np.nan
    np.testing.assert_array_equal(magicpig.project_signs_fast(x, p), magicpig.project_signs(x, p))


def test_chunked_step_equals_the_whole_sequence():
    """`chunked_step` (the form that scales to 1M keys) against `run_stack` on a sequence that
    fits: identical masks chunk by chunk, the same output."""
    wl = workloads.magicpig(seed=64, dtype="bf16", B=1, Hq=8, Hkv=2, S=1500, D=128, sink=6, window=20,
                            lsh_l=30, lsh_k=6, n_clusters=8)
    proj = wl.stack[-1][1]["projection"]
    ref_mask, ref_out, _ = _oracle(wl, {})
    masks = {}
    out, st = magicpig.chunked_step(wl.stack[-1][1], 6, 20, wl.q,
                                    lambda a, b: (wl.k[:, :, a:b], wl.v[:, :, a:b]), 1500, 400, "bf16",
                                    proj, wl.scaling, on_chunk=lambda a, b, m, c: masks.__setitem__(a, m))
    np.testing.assert_array_equal(np.concatenate([masks[a] for a in sorted(masks)], axis=-1), ref_mask)
    np.testing.assert_allclose(out, ref_out, atol=4e-3, rtol=1e-2)
    # handing a chunk its matches instead of its signatures changes nothing
    def _m(a, b):
        return ref_mask[..., a:b] != 0

    out2, _ = magicpig.chunked_step(wl.stack[-1][1], 6, 20, wl.q,
                                    lambda a, b: (wl.k[:, :, a:b], wl.v[:, :, a:b]), 1500, 400, "bf16",
                                    proj, wl.scaling, known_match=lambda a, b: None if a == 400 else _m(a, b))
    np.testing.assert_array_equal(out2, out)


# ------------------------------------------------------------------ CPU: arithmetic shortcuts of the kernels
def _rn(x, bits):
    """Round a positive Fraction to `bits` significant bits, ties to even (no range limits)."""
    from fractions import Fraction
    import math

    if x == 0:
        return Fraction(0)
    e = math.floor(math.log2(x))
    while Fraction(2) ** e > x:
        e -= 1
    while Fraction(2) ** (e + 1) <= x:
        e += 1
    scale = Fraction(2) ** (e - bits + 1)
    n = x / scale
    lo = n.numerator // n.denominator
    rem = n - lo
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and lo % 2 == 1):
        lo += 1
    return lo * scale


def test_reciprocal_division_of_bf16_values_is_exact():
    """The probability kernel divides a bf16 value by a bf16 value as q = RN(x*y), r = x - q*d,
    RN(q + r*y) with y = RN(1/d) in float32, then rounds to bf16.  For every pair of bf16
    significands this equals the IEEE float32 quotient rounded to bf16 (signs and exponents
    factor out of every step)."""
    from fractions import Fraction

    for d in range(128, 256):
        y = _rn(Fraction(1, d), 24)
        for x in range(128, 256):
            q = _rn(x * y, 24)
            r = x - q * d
            assert abs(r) == _rn(abs(r), 24)  # the fma residual is exact
            q2 = q + r * y
            assert q2 > 0
            got = _rn(_rn(q2, 24), 8)
            want = _rn(_rn(Fraction(x, d), 24), 8)
            assert got == want, (x, d)


@pytest.mark.gpu
@pytest.mark.parametrize("L,S,centred", [(75, 20000, True), (33, 9000, True), (75, 5000, False)])
def test_gpu_signatures_from_tensor_cores_equal_the_fixed_order_kernel(L, S, centred):
    """`sah_lsh_key_sign_tc` (tcgen05 projections, near-zero ones redone in the fixed order) writes
    bit for bit the signature rows of `sah_lsh_key_sign`, padding bytes included; a short range
    is also checked against the CPU restatement."""
    import torch
    from sparse_attention_hub import _native

    lib = _native.load()
    dev = "cuda:0"
    B, Hkv, D, K, cap = 2, 2, 128, 8, S + 64
    gen = torch.Generator(device=dev).manual_seed(5 + L)
    keys = (torch.randn((B, Hkv, cap, D), generator=gen, device=dev) * 0.7 + 0.3).to(torch.bfloat16)[:, :, :S]
    proj = torch.randn((D + 1, L * K), generator=gen, device=dev).to(torch.bfloat16)
    mean = keys.float().mean(dim=2).to(torch.bfloat16).contiguous() if centred else None
    norms = torch.zeros((B, Hkv, cap), dtype=torch.float32, device=dev)
    max_norm = torch.zeros(1, dtype=torch.int32, device=dev)
    st = _native.stream_of(torch.device(dev))
    kargs = (keys.data_ptr(), _native.SAH_BF16, keys.stride(0), keys.stride(1), keys.stride(2), B, Hkv)
    _native.check(lib.sah_lsh_key_stats(*kargs, 0, S, D, _native.ptr(mean), cap, norms.data_ptr(),
                                        max_norm.data_ptr(), 148, st), "sah_lsh_key_stats")
    pitch = (L + 15) // 16 * 16
    want = torch.full((B, Hkv, cap, pitch), 0xAA, dtype=torch.uint8, device=dev)
    got = torch.full_like(want, 0x55)
    _native.check(lib.sah_lsh_key_sign(*kargs, 0, S, D, _native.ptr(mean), norms.data_ptr(), max_norm.data_ptr(),
                                       proj.data_ptr(), L, K, cap, want.data_ptr(), st), "sah_lsh_key_sign")
    nbytes = int(lib.sah_lsh_key_sign_tc_ws_bytes(B, Hkv, S))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _native.check(lib.sah_lsh_key_sign_tc(keys.data_ptr(), keys.stride(0), keys.stride(1), keys.stride(2), B, Hkv,
                                          0, S, D, _native.ptr(mean), norms.data_ptr(), max_norm.data_ptr(),
                                          proj.data_ptr(), L, K, cap, got.data_ptr(), ws.data_ptr(), nbytes, 148,
                                          st), "sah_lsh_key_sign_tc")
    torch.cuda.synchronize()
    redone, err = ws[:8].view(torch.int32).tolist()
    assert err == 0 and 0 <= redone <= (nbytes - 16) // 16
    assert torch.equal(got[:, :, :S], want[:, :, :S])
    assert bool((got[:, :, S:] == 0x55).all())  # rows past the range are not touched
    # a few hundred keys against the CPU restatement of the reference's transform and projection
    n = 300
    k_np = keys[:, :, :n].float().cpu().numpy()
    m_np = None if mean is None else mean.float().cpu().numpy()
    M = np.float32(max_norm.view(torch.float32).item())
    nk = norms[:, :, :n].cpu().numpy()
    np.testing.assert_array_equal(nk, magicpig.norms(magicpig.centred(
        k_np, None if m_np is None else m_np[:, :, None, :], "bf16"), "bf16"))
    codes = magicpig.key_codes(k_np, m_np, nk, M, proj.float().cpu().numpy(), L, K, "bf16")
    np.testing.assert_array_equal(got[:, :, :n, :L].cpu().numpy().astype(np.int64), codes)
