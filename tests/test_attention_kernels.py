"""The two bfloat16 attention kernels (mma.sync over 16-key tiles, tcgen05 over 128-key tiles)
against the CPU restatement of the reference on the same masks: unit weights, per-entry weights,
MagicPig weights evaluated in the kernel, attention-mask bias with several queries, sink logits,
sixteen mask rows per group, lists shorter than one tile and lists of many tiles per CTA, and
strided K/V views (a slice of a longer cache)."""

import numpy as np
import pytest
import torch

import workloads
from oracle import attention as o_attention
from oracle import stacks
from sparse_attention_hub.sparse_attention import Mask
from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import (
    attention_wait_errors,
    get_masked_attention_output,
    native_masked_attention,
    select_attention_kernel,
)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-2


@pytest.fixture(params=["mma", "umma"])
def kernel(request):
    prev = select_attention_kernel(request.param)
    yield request.param
    select_attention_kernel(prev)
    assert attention_wait_errors() == 0, "a bounded wait inside the attention kernel ran out"


def _dense_mask_case(seed, B, Hq, Hkv, S, D, density, weighted, Sq=1):
    wl = workloads.sink_local_fp32(seed=seed, B=B, Hq=Hq, Hkv=Hkv, S=S, D=D, Sq=Sq)
    rng = np.random.default_rng(seed)
    q, k, v = (workloads.to_dtype(a, "bf16") for a in (wl.q, wl.k, wl.v))
    sel = rng.random((B, Hq, Sq, S)) < density
    vals = rng.uniform(0.05, 1.0, sel.shape) if weighted else np.ones(sel.shape)
    dense = np.where(sel, vals, 0.0)
    dense[..., :4] = 1.0
    dense = workloads.to_dtype(dense.astype(np.float32), "bf16")
    return wl, q, k, v, dense


@pytest.mark.parametrize("S,density,weighted", [(100, 0.3, False), (700, 0.15, True), (9000, 0.4, False),
                                                (40000, 0.5, True)])
def test_dense_mask_attention(kernel, S, density, weighted):
    wl, q, k, v, dense = _dense_mask_case(61 + S % 7, 2, 8, 2, S, 128, density, weighted)
    tq, tk, tv = (workloads.to_torch(a, "bf16", DEV) for a in (q, k, v))
    m = Mask.create_mask_from_dense_mask(dense.shape, workloads.to_torch(dense, "bf16", DEV), torch.bfloat16)
    out = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), m)
    ref = o_attention.masked_attention(q, k, v, dense, wl.scaling, "bf16")
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=TOL, rtol=TOL)


def test_sixteen_rows_and_strided_cache(kernel):
    wl, q, k, v, dense = _dense_mask_case(71, 1, 16, 1, 3000, 128, 0.25, True)
    tq = workloads.to_torch(q, "bf16", DEV)
    # K and V are the first 3000 rows of a cache of 4096: the batch/head strides are not S * D
    cache_k = torch.zeros((1, 1, 4096, 128), dtype=torch.bfloat16, device=DEV)
    cache_v = torch.zeros_like(cache_k)
    cache_k[:, :, :3000] = workloads.to_torch(k, "bf16", DEV)
    cache_v[:, :, :3000] = workloads.to_torch(v, "bf16", DEV)
    m = Mask.create_mask_from_dense_mask(dense.shape, workloads.to_torch(dense, "bf16", DEV), torch.bfloat16)
    out = native_masked_attention(tq, cache_k[:, :, :3000], cache_v[:, :, :3000], None, None,
                                  float(wl.scaling), m)
    ref = o_attention.masked_attention(q, k, v, dense, wl.scaling, "bf16")
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=TOL, rtol=TOL)


def test_several_queries_with_bias_and_sink_logits(kernel):
    wl = workloads.sink_local_fp32(seed=73, B=2, Hq=4, Hkv=2, S=2600, D=128, sink=8, window=300, Sq=3)
    rng = np.random.default_rng(5)
    am = np.zeros((2, 1, 3, 2600), dtype=np.float32)
    for i in range(3):  # causal over the last three positions, plus a few blocked keys
        am[:, :, i, 2600 - 2 + i:] = -np.inf
    am[:, :, :, rng.integers(0, 2500, 40)] = -np.inf
    sinks = rng.normal(size=4).astype(np.float32)
    q, k, v = (workloads.to_dtype(a, "bf16") for a in (wl.q, wl.k, wl.v))
    ra = workloads.research_attention(wl.stack, "bf16", DEV)
    tq, tk, tv = (workloads.to_torch(a, "bf16", DEV) for a in (q, k, v))
    tam = workloads.to_torch(am, "bf16", DEV)
    mask = ra.build_mask(tq, tk, tv, tam, float(wl.scaling), 0.0, {}, layer_idx=0)
    out = get_masked_attention_output(None, tq, tk, tv, tam, torch.from_numpy(sinks).to(DEV),
                                      float(wl.scaling), 0.0, mask)
    _, ref, _ = stacks.run_stack(wl.stack, q, k, v, wl.scaling, "bf16", attention_mask=am, sinks=sinks)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=TOL, rtol=TOL)


@pytest.mark.parametrize("S", [3000, 50000])
def test_magicpig_weights_inside_the_kernel(kernel, S):
    wl = workloads.magicpig(seed=75, B=1, Hq=8, Hkv=2, S=S, D=128, dtype="bf16")
    ra = workloads.research_attention(wl.stack, "bf16", DEV)
    q, k, v = (workloads.to_torch(a, "bf16", DEV) for a in (wl.q, wl.k, wl.v))
    meta = {"projections": {0: workloads.to_torch(wl.stack[-1][1]["projection"], "bf16", DEV)}}
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    _, ref, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                 meta={"lsh_projection": wl.stack[-1][1]["projection"]})
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=TOL, rtol=TOL)


def test_bounded_wait_runs_out_and_reports_without_hanging():
    """Every mbarrier wait of the tcgen05 kernels is bounded.  `sah_wait_selftest` waits 2 ms for an
    arrival that never comes: the error word is set, the measured wait is about the limit, the
    kernel returns, and the next attention call on the same context works."""
    from sparse_attention_hub import _native

    lib = _native.load()
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    _native.check(lib.sah_wait_selftest(2000, err.data_ptr(), waited.data_ptr(),
                                        _native.stream_of(torch.device(DEV))), "sah_wait_selftest")
    torch.cuda.synchronize()
    assert int(err.item()) != 0
    assert 2_000_000 <= int(waited.item()) < 50_000_000
    prev = select_attention_kernel("umma")
    try:
        wl, q, k, v, dense = _dense_mask_case(77, 1, 8, 2, 2000, 128, 0.3, False)
        tq, tk, tv = (workloads.to_torch(a, "bf16", DEV) for a in (q, k, v))
        m = Mask.create_mask_from_dense_mask(dense.shape, workloads.to_torch(dense, "bf16", DEV), torch.bfloat16)
        out = native_masked_attention(tq, tk, tv, None, None, float(wl.scaling), m)
        ref = o_attention.masked_attention(q, k, v, dense, wl.scaling, "bf16")
        np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=TOL, rtol=TOL)
    finally:
        select_attention_kernel(prev)
