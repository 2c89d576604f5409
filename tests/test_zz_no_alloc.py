"""`sah_masked_attention_static`: masked attention for callers that cannot allocate.

A host that had its device memory partitioned once at start-up, or that may not
allocate from the CUDA driver after initialisation, cannot give the library the
work lists and partial buffers that plan + gather attention need.  The static
entry point keeps them in a device array inside the library image.  This test
calls it through the C ABI, two calls in a row on the same array (different
queries and a different mask the second time, so that stale contents would
show), and compares each output with the regular entry points, which take
caller-provided workspace, and with the CPU restatement of the reference.  It also checks that a problem beyond the built-in
limits is refused with a clear message instead of being run.
"""

import ctypes

import numpy as np
import pytest
import torch

import workloads
from oracle import stacks
from sparse_attention_hub import _native
from sparse_attention_hub.sparse_attention import Mask
from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import native_masked_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static_attention(q, k, v, mask: Mask, scaling: float) -> torch.Tensor:
    lib = _native.load()
    B, Hq, Sq, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    nb = mask.native_bits()
    assert nb.data is None, "the static entry point takes unit-weight masks"
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    status = lib.sah_masked_attention_static(
        nb.bits.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), _native.dtype_code(q.dtype),
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), B, Hq, Hkv, Sq, S, nb.words, D, float(scaling),
        None, 0, 0, 0, None, _native.sm_count(q.device), out.data_ptr(),
        _native.stream_of(q.device))
    _native.check(status, "sah_masked_attention_static")
    return out


@pytest.mark.parametrize("dtype,tol", [("bf16", 2e-2), ("f32", 1e-4)])
def test_static_scratch_matches_workspace_path_twice(dtype, tol):
    seeds = (61, 62)
    for call, seed in enumerate(seeds):
        wl = workloads.sink_local_fp32(seed=seed, B=2, Hq=8, Hkv=2, S=3000 + 500 * call, D=128,
                                       sink=16 + call, window=64)
        ra = workloads.research_attention(wl.stack, dtype, DEV)
        q, k, v = (workloads.to_torch(workloads.to_dtype(a, dtype), dtype, DEV)
                   for a in (wl.q, wl.k, wl.v))
        mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, {}, layer_idx=0)
        want = native_masked_attention(q, k, v, None, None, float(wl.scaling), mask)
        got = _static_attention(q, k, v, mask, float(wl.scaling))
        torch.cuda.synchronize()
        np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(),
                                   atol=tol, rtol=tol)
        # and with the CPU restatement of the reference on the same inputs
        qn, kn, vn = (workloads.to_dtype(a, dtype) for a in (wl.q, wl.k, wl.v))
        _, ref_out, _ = stacks.run_stack(wl.stack, qn, kn, vn, wl.scaling, dtype)
        np.testing.assert_allclose(got.float().cpu().numpy(), ref_out, atol=tol, rtol=tol)


def test_static_scratch_rejects_oversized_problem():
    lib = _native.load()
    B, Hq, Hkv, Sq, S, D = 4, 32, 8, 1, 65536, 128  # 32 groups x 65536 keys = 2^21 slots
    q = torch.zeros((B, Hq, Sq, D), dtype=torch.bfloat16, device=DEV)
    kv = torch.zeros((1, 1, 8, D), dtype=torch.bfloat16, device=DEV)  # never dereferenced
    bits = torch.zeros(16, dtype=torch.int32, device=DEV)
    out = torch.zeros((B, Sq, Hq, D), dtype=torch.bfloat16, device=DEV)
    status = lib.sah_masked_attention_static(
        bits.data_ptr(), q.data_ptr(), kv.data_ptr(), kv.data_ptr(), _native.SAH_BF16,
        q.stride(0), q.stride(1), q.stride(2), 0, 0, D, 0, 0, D, B, Hq, Hkv, Sq, S, S // 32, D,
        1.0, None, 0, 0, 0, None, 148, out.data_ptr(), _native.stream_of(q.device))
    assert status == 4  # SAH_ERR_WORKSPACE
    msg = lib.sah_last_error().decode()
    assert "built-in scratch" in msg and "2097152" in msg
