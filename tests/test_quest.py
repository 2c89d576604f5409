"""Quest page top-k: numpy restatement vs the reference's fixtures (CPU), CUDA path vs both (GPU).

Page scores are sums of dtype-rounded products taken in the reference's CPU reduction order; the
fixtures hold the reference's own page scores, which the restatement and the kernel reproduce bit
for bit in bfloat16 and float32, and with them the chosen pages.
"""

import numpy as np
import pytest

from oracle import mask_ops, quest, stacks
import workloads

from conftest import load_golden

CASES = (("quest_bf16", "bf16", 81, 1000, 128, 16, 0.1, False),
         ("quest_f32", "f32", 82, 768, 64, 32, 96, False),
         ("quest_bf16_masked", "bf16", 83, 1024, 128, 16, 0.1, True))


def _case(name, dtype, seed, S, D, page, heavy):
    wl = workloads.oracle_topk(seed=seed, dtype=dtype, B=2, Hq=8, Hkv=2, S=S, D=D, sink=16, window=32)
    stack = [("sink", {"sink_size": 16}), ("local", {"window_size": 32}),
             ("quest_topk", {"heavy_size": heavy, "page_size": page})]
    return wl, stack


@pytest.mark.parametrize("name,dtype,seed,S,D,page,heavy,masked", CASES)
def test_restatement_against_reference(name, dtype, seed, S, D, page, heavy, masked):
    g = load_golden(name)
    wl, stack = _case(name, dtype, seed, S, D, page, heavy)
    am = g["attention_mask"] if masked else None
    mask, out, meta = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, dtype, attention_mask=am)
    sc = meta["quest_page_scores"]
    gated = sc < -1e30            # the fixture's scores are taken before the validity gate
    np.testing.assert_array_equal(np.where(gated, g["page_scores"], sc), g["page_scores"])
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])
    np.testing.assert_allclose(out, g["out"], atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)


def test_restatement_three_query_positions_under_a_causal_mask():
    """Reference fixture with three query positions under an HF causal mask: page scores, index
    sets, weights and output of the restatement are the reference's."""
    g = load_golden("quest_bf16_sq3_causal")
    wl = workloads.oracle_topk(seed=84, dtype="bf16", B=2, Hq=8, Hkv=2, S=640, D=128, sink=16, window=32, Sq=3)
    stack = [("sink", {"sink_size": 16}), ("local", {"window_size": 32}),
             ("quest_topk", {"heavy_size": 0.1, "page_size": 16})]
    mask, out, meta = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, "bf16",
                                       attention_mask=g["attention_mask"])
    sc = meta["quest_page_scores"]
    gated = sc < -1e30
    np.testing.assert_array_equal(np.where(gated, g["page_scores"], sc), g["page_scores"])
    idx, ptr, data = mask_ops.to_csr(mask)
    np.testing.assert_array_equal(idx, g["idx"])
    np.testing.assert_array_equal(ptr, g["ptr"])
    np.testing.assert_array_equal(data, g["data"])
    np.testing.assert_allclose(out, g["out"], atol=2e-2, rtol=2e-2)


def test_row_sum_order_against_torch():
    """The restated reduction order is torch's on this machine, for both dtypes and odd lengths."""
    import torch
    torch.manual_seed(3)
    for D in (128, 64, 100, 40, 256):
        x = torch.randn(3000, D)
        np.testing.assert_array_equal(quest.row_sum(x.numpy(), "f32"), x.sum(-1).numpy())
        xb = x.to(torch.bfloat16)
        np.testing.assert_array_equal(quest.row_sum(xb.float().numpy(), "bf16"), xb.sum(-1).float().numpy())


def test_config_and_rules_cpu():
    import torch
    from sparse_attention_hub.sparse_attention import Mask, QuestTopKMasker, QuestTopKMaskerConfig

    with pytest.raises(ValueError):
        QuestTopKMaskerConfig(heavy_size=0.1, page_size=0)
    with pytest.raises(ValueError):
        QuestTopKMaskerConfig(heavy_size=0.1, page_size=16, label_bits=17)
    with pytest.raises(ValueError):
        QuestTopKMasker.create_from_config(object())
    m = QuestTopKMasker.create_from_config(QuestTopKMaskerConfig(heavy_size=64, page_size=16))
    q, k = torch.zeros(1, 2, 1, 8), torch.zeros(1, 2, 48, 8)
    prev = Mask.create_empty_mask((1, 2, 1, 48), torch.float32, torch.device("cpu"))
    assert m.add_mask(k, q, k, None, 1.0, 0.0, {}, prev).is_full_mask()      # S <= heavy
    m = QuestTopKMasker.create_from_config(QuestTopKMaskerConfig(heavy_size=8, page_size=16, label_bits=8))
    with pytest.raises(NotImplementedError):
        m.add_mask(k, q, k, None, 1.0, 0.0, {}, prev)


# ------------------------------------------------------------------ GPU
def _native_stack(wl, stack, am, meta, with_out=True):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    dev = "cuda:0"
    ra = workloads.research_attention(stack, wl.dtype, dev)
    q, k, v = (workloads.to_torch(a, wl.dtype, dev) for a in (wl.q, wl.k, wl.v))
    amt = None if am is None else workloads.to_torch(am, wl.dtype, dev)
    mask = ra.build_mask(q, k, v, amt, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = None
    if with_out:
        out = get_masked_attention_output(None, q, k, v, amt, None, float(wl.scaling), 0.0, mask)
        out = out.float().cpu().numpy()
    torch.cuda.synchronize()
    idx, ptr, data = mask.get_index_mask()
    return (idx.cpu().numpy(), ptr.cpu().numpy(), data.float().cpu().numpy()), out


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype,seed,S,D,page,heavy,masked", CASES)
def test_gpu_stack_against_reference(name, dtype, seed, S, D, page, heavy, masked):
    g = load_golden(name)
    wl, stack = _case(name, dtype, seed, S, D, page, heavy)
    am = g["attention_mask"] if masked else None
    got, out = _native_stack(wl, stack, am, {})
    np.testing.assert_array_equal(got[0], g["idx"])
    np.testing.assert_array_equal(got[1], g["ptr"])
    np.testing.assert_array_equal(got[2], g["data"])
    np.testing.assert_allclose(out, g["out"], atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,S,D,page,heavy,Sq", [("bf16", 8192, 128, 64, 0.05, 1), ("f32", 3000, 64, 48, 200, 2),
                                                     ("bf16", 4100, 72, 20, 0.1, 1), ("f32", 2048, 40, 16, 0.2, 1)])
def test_gpu_page_scores_and_mask_against_restatement(dtype, S, D, page, heavy, Sq):
    """Longer rows, page sizes that do not divide 32, head dimensions with a vector tail."""
    import torch
    from sparse_attention_hub import _native

    wl = workloads.oracle_topk(seed=S + D, dtype=dtype, B=1, Hq=8, Hkv=4, S=S, D=D, sink=8, window=24, Sq=Sq)
    stack = [("sink", {"sink_size": 8}), ("local", {"window_size": 24}),
             ("quest_topk", {"heavy_size": heavy, "page_size": page})]
    ref_mask, ref_out, meta = stacks.run_stack(stack, wl.q, wl.k, wl.v, wl.scaling, dtype)
    # the score kernel on its own
    lib = _native.load()
    dev = torch.device("cuda:0")
    q, k = (workloads.to_torch(a, dtype, dev) for a in (wl.q, wl.k))
    P = -(-S // page)
    pmin = torch.empty((1, 4, D // 8, P, 8), dtype=q.dtype, device=dev)   # [B, Hkv, D/8, pages, 8]
    pmax = torch.empty_like(pmin)
    st = _native.stream_of(dev)
    code = _native.dtype_code(q.dtype)
    _native.check(lib.sah_quest_page_minmax(k.data_ptr(), code, k.stride(0), k.stride(1), k.stride(2), 1, 4, S, D,
                                            page, 0, P, pmin.data_ptr(), pmax.data_ptr(), st), "minmax")
    lo, hi = quest.page_min_max(np.asarray(wl.k, np.float32), page)
    np.testing.assert_array_equal(pmin.permute(0, 1, 3, 2, 4).reshape(1, 4, P, D).float().cpu().numpy(), lo)
    np.testing.assert_array_equal(pmax.permute(0, 1, 3, 2, 4).reshape(1, 4, P, D).float().cpu().numpy(), hi)
    sc = torch.empty((1, 8, Sq, P), dtype=q.dtype, device=dev)
    _native.check(lib.sah_quest_scores(q.data_ptr(), code, q.stride(0), q.stride(1), q.stride(2), pmin.data_ptr(),
                                       pmax.data_ptr(), P, 1, 8, 4, Sq, S, D, page, None, 0, 0, 0,
                                       sc.data_ptr(), st), "scores")
    np.testing.assert_array_equal(sc.float().cpu().numpy(), meta["quest_page_scores"])
    attend = D in (64, 128)     # the attention kernels take head dimensions 64 and 128
    got, out = _native_stack(wl, stack, None, {}, with_out=attend)
    ri, rp, rd = mask_ops.to_csr(ref_mask)
    np.testing.assert_array_equal(got[0], ri)
    np.testing.assert_array_equal(got[1], rp)
    if attend:
        np.testing.assert_allclose(out, ref_out, atol=1e-4 if dtype == "f32" else 2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_gpu_appended_keys_update_only_their_pages():
    """A second call with more keys reuses the cached page bounds and gives what a fresh call gives."""
    import torch

    wl = workloads.oracle_topk(seed=91, dtype="bf16", B=2, Hq=8, Hkv=2, S=1500, D=128, sink=8, window=24)
    stack = [("sink", {"sink_size": 8}), ("local", {"window_size": 24}),
             ("quest_topk", {"heavy_size": 0.1, "page_size": 32})]
    dev = "cuda:0"
    ra = workloads.research_attention(stack, "bf16", dev)
    q, k, v = (workloads.to_torch(a, "bf16", dev) for a in (wl.q, wl.k, wl.v))
    meta: dict = {}
    for n in (600, 601, 640, 1500):        # growth inside a page, across pages, and past the capacity
        mask = ra.build_mask(q, k[:, :, :n], v[:, :, :n], None, float(wl.scaling), 0.0, meta, layer_idx=0)
        fresh = ra.build_mask(q, k[:, :, :n], v[:, :, :n], None, float(wl.scaling), 0.0, {}, layer_idx=0)
        assert meta["quest_pages"][0]["n_keys"] == n
        a, b = mask.get_index_mask(), fresh.get_index_mask()
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
        ref_mask, _, _ = stacks.run_stack(stack, wl.q, wl.k[:, :, :n], wl.v[:, :, :n], wl.scaling, "bf16")
        np.testing.assert_array_equal(a[0].cpu().numpy(), mask_ops.to_csr(ref_mask)[0])
