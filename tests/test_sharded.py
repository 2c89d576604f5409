"""Sequence-sharded decode.

CPU: the shard planner, the in-process collectives, and -- as two gloo ranks -- the numpy
restatement of the sharded algorithm (global sizes, global key mean / maximum norm, global
top-k with ties to the lowest column, partial softmax merge) against the unsharded
restatement, together with the product's `DistComm` wrappers.
GPU: the CUDA path with the ranks run as threads of one process on one device
(`ThreadComm`: only host threads wait on each other), against the unsharded CUDA path and
the restatement.  The union of the ranks' local masks must be the unsharded mask exactly.
"""

import os
import socket
import threading

import numpy as np
import pytest

from oracle import mask_ops, sharded as o_sharded, stacks
import workloads
from sparse_attention_hub.sparse_attention.research_attention.sharded import (
    ThreadComm,
    plan_shards,
)


def _magicpig_wl(dtype="bf16", S=1000, Sq=1, seed=71):
    return workloads.magicpig(seed=seed, dtype=dtype, B=2, Hq=4, Hkv=2, S=S, D=64, sink=5, window=40,
                              lsh_l=12, lsh_k=4, Sq=Sq, n_clusters=4)


def _hash_wl(S=1000, seed=72):
    return workloads.hashattention_bf16(seed=seed, B=2, Hq=4, Hkv=2, S=S, D=64, sink=5, window=40,
                                        heavy=0.05, hidden=32, layers=2)


def _oracle_wl(dtype="bf16", S=1000, seed=74):
    wl = workloads.oracle_topk(seed=seed, dtype=dtype, B=2, Hq=4, Hkv=2, S=S, D=64, sink=5, window=40, heavy=0.05)
    # duplicate a block of keys so that equal scores straddle the shard boundaries
    wl.k[:, :, 300:700] = wl.k[:, :, 100:500]
    return wl


PQ_CENT, PQ_ITERS = 16, 5


def _pq_wl(S=1200, seed=76):
    wl = workloads.pqcache(seed=seed, dtype="bf16", B=2, Hq=4, Hkv=2, S=S, D=64, sink=40, window=24, heavy=60,
                           group_factor=8, bits=4, kmeans_iter=PQ_ITERS, n_clusters=8)
    # a block of duplicated keys: equal scores on both sides of the shard boundaries
    wl.k[:, :, 500:800] = wl.k[:, :, 100:400]
    return wl


def _pq_draws(wl):
    """Initial centres and re-seed draws handed to every implementation (the reference draws them
    with torch.randperm / torch.randint)."""
    B, Hkv, S = wl.k.shape[0], wl.k.shape[1], wl.k.shape[2]
    prm = wl.stack[-1][1]
    groups, n = B * Hkv * prm["pq_group_factor"], S - prm["init_offset"]
    init = workloads.pq_init_indices(77, groups, n, PQ_CENT)
    reseed = np.random.default_rng(78).integers(0, n, size=(PQ_ITERS, groups, PQ_CENT)).astype(np.int64)
    return init, reseed


def _oracle_meta(wl):
    last = wl.stack[-1]
    if last[0] == "pq_topk":
        init, reseed = _pq_draws(wl)
        return {"pq_init_indices": init, "pq_reseed_indices": reseed}
    return {"lsh_projection": last[1]["projection"]} if last[0] == "magicpig" else {}


def test_plan_shards_covers_the_sequence_in_whole_words():
    for total, world in ((1048576, 8), (1000, 4), (33, 2), (31, 4), (0, 2)):
        plan = plan_shards(total, world)
        assert len(plan) == world and plan[0][0] == 0 and plan[-1][1] == total
        for (b0, e0), (b1, e1) in zip(plan, plan[1:]):
            assert e0 == b1 and b0 <= e0
        assert all(b % 32 == 0 for b, e in plan if e > b)
        assert plan == o_sharded.plan_shards(total, world)


def test_thread_comm_collectives():
    import torch

    comms = ThreadComm.create(3)
    out = [None] * 3

    def work(r):
        c = comms[r]
        a = c.all_reduce_sum_(torch.tensor([float(r + 1), 1.0]))
        m = c.all_reduce_max_(torch.tensor([r * 10]))
        g = c.all_gather(torch.tensor([r, r]))
        out[r] = (a, m, g)

    ts = [threading.Thread(target=work, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for a, m, g in out:
        assert a.tolist() == [6.0, 3.0] and m.tolist() == [20] and g.tolist() == [[0, 0], [1, 1], [2, 2]]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank: int, world: int, port: int, results) -> None:
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sparse_attention_hub.sparse_attention.research_attention.sharded import DistComm

        c = DistComm()
        assert c.all_reduce_sum_(torch.tensor([rank + 1.0])).item() == sum(range(1, world + 1))
        assert c.all_reduce_max_(torch.tensor([rank])).item() == world - 1
        assert c.all_gather(torch.tensor([rank, 7])).tolist() == [[r, 7] for r in range(world)]

        comm = o_sharded.TorchComm()
        ok = True
        for wl, dtype in ((_magicpig_wl("bf16"), "bf16"), (_magicpig_wl("f32", S=700, Sq=2), "f32"),
                          (_hash_wl(), "bf16"), (_oracle_wl("bf16"), "bf16")):
            S = wl.k.shape[2]
            b, e = o_sharded.plan_shards(S, world)[rank]
            ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype,
                                                    meta=_oracle_meta(wl))
            mask, out, _ = o_sharded.run_sharded(wl.stack, wl.q, wl.k[:, :, b:e], wl.v[:, :, b:e], wl.scaling,
                                                 dtype, o_sharded.Shard(b, S, comm), _oracle_meta(wl))
            ok &= bool(np.array_equal(mask, ref_mask[..., b:e]))
            ok &= bool(np.allclose(out, ref_out, atol=2e-2 if dtype == "bf16" else 1e-5, rtol=1e-2))
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_sharded_restatement_two_gloo_ranks():
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_gloo_rank, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}


# ------------------------------------------------------------------ GPU: ranks as threads on one device
def _native_unsharded(wl, meta):
    import torch
    from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import get_masked_attention_output

    dev = "cuda:0"
    ra = workloads.research_attention(wl.stack, wl.dtype, dev)
    q, k, v = (workloads.to_torch(a, wl.dtype, dev) for a in (wl.q, wl.k, wl.v))
    mask = ra.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
    out = get_masked_attention_output(None, q, k, v, None, None, float(wl.scaling), 0.0, mask)
    torch.cuda.synchronize()
    return mask.get_dense_mask().float().cpu().numpy(), out.float().cpu().numpy()


def _native_sharded(wl, world, make_meta):
    import torch
    from sparse_attention_hub.sparse_attention.research_attention.sharded import SequenceShardedAttention

    dev = "cuda:0"
    S = wl.k.shape[2]
    plan = plan_shards(S, world)
    comms = ThreadComm.create(world)
    results, errors = [None] * world, []

    def rank_fn(r):
        try:
            torch.cuda.set_device(0)
            b, e = plan[r]
            ra = workloads.research_attention(wl.stack, wl.dtype, dev)
            sa = SequenceShardedAttention(ra, comms[r], b, S)
            q = workloads.to_torch(wl.q, wl.dtype, dev)
            k = workloads.to_torch(wl.k[:, :, b:e], wl.dtype, dev)
            v = workloads.to_torch(wl.v[:, :, b:e], wl.dtype, dev)
            meta = make_meta(dev)
            mask = sa.build_mask(q, k, v, None, float(wl.scaling), 0.0, meta, layer_idx=0)
            out, _ = sa.custom_attention(None, q, k, v, None, float(wl.scaling), 0.0,
                                         sparse_meta_data=meta, layer_idx=0)
            torch.cuda.synchronize()
            dense = None if (mask.is_full or mask.is_empty) else mask.get_dense_mask().float().cpu().numpy()
            results[r] = (dense, out.float().cpu().numpy())
        except BaseException as exc:  # a failed rank must not leave the others at a barrier
            errors.append(exc)
            for c in comms:
                c._barrier.abort()

    threads = [threading.Thread(target=rank_fn, args=(r,)) for r in range(world)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    if errors:
        raise errors[0]
    return plan, results


def _proj_meta(wl):
    def make(dev):
        import torch

        last = wl.stack[-1]
        if last[0] == "pq_topk":
            init, reseed = _pq_draws(wl)
            return {"pq_init_indices": {0: torch.from_numpy(init)}, "pq_reseed_indices": {0: torch.from_numpy(reseed)}}
        if last[0] != "magicpig":
            return {}
        return {"projections": {0: workloads.to_torch(last[1]["projection"], wl.dtype, dev)}}
    return make


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["magicpig_bf16", "magicpig_f32_sq2", "hash_bf16", "oracle_bf16", "oracle_f32",
                                  "pq_bf16"])
@pytest.mark.parametrize("world", [2, 4])
def test_gpu_sharded_equals_unsharded(case, world):
    wl = {"magicpig_bf16": lambda: _magicpig_wl("bf16"),
          "magicpig_f32_sq2": lambda: _magicpig_wl("f32", S=700, Sq=2),
          "hash_bf16": _hash_wl, "oracle_bf16": lambda: _oracle_wl("bf16"),
          "oracle_f32": lambda: _oracle_wl("f32", S=900), "pq_bf16": _pq_wl}[case]()
    dtype = wl.dtype
    full_mask, full_out = _native_unsharded(wl, _proj_meta(wl)("cuda:0"))
    plan, results = _native_sharded(wl, world, _proj_meta(wl))
    union = np.concatenate([results[r][0] for r in range(world)], axis=-1)
    np.testing.assert_array_equal(union, full_mask)
    ref_mask, ref_out, _ = stacks.run_stack(wl.stack, wl.q, wl.k, wl.v, wl.scaling, dtype, meta=_oracle_meta(wl))
    np.testing.assert_array_equal(union, ref_mask)
    tol = 2e-2 if dtype == "bf16" else 1e-4
    per_row = {f"rank{r}": (np.abs(results[r][1] - full_out).max(axis=-1).reshape(-1).round(4).tolist(),
                            np.abs(results[r][1] - ref_out).max(axis=-1).reshape(-1).round(4).tolist())
               for r in range(world)}
    for r in range(world):
        np.testing.assert_allclose(results[r][1], full_out, atol=tol, rtol=2e-2, err_msg=str(per_row))
        np.testing.assert_allclose(results[r][1], ref_out, atol=tol, rtol=2e-2, err_msg=str(per_row))


@pytest.mark.gpu
def test_gpu_unshardable_masker_refuses_a_shard():
    wl = workloads.oracle_adaptive(seed=73, dtype="bf16", B=1, Hq=4, Hkv=2, S=512, D=64, sink=4, window=8)
    with pytest.raises(NotImplementedError):
        _native_sharded(wl, 2, lambda dev: {})


# ------------------------------------------------------------------ GPUs: the peer-memory exchange
def _nccl_rank(rank: int, world: int, port: int, results) -> None:
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from sparse_attention_hub.sparse_attention.research_attention.sharded import DistComm, PeerExchange
        from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import merge_attention_partials

        comm = DistComm()
        B, Hq, Sq, D = 2, 8, 3, 128
        rows = B * Hq * Sq
        ex = PeerExchange(comm, B, Hq, Sq, D, torch.device("cuda", rank))
        sinks = torch.linspace(-1.0, 1.0, Hq, device="cuda")
        ok = True
        for step in range(5):  # both parities several times
            gen = torch.Generator(device="cuda").manual_seed(100 * step + rank)
            part = torch.randn((rows, D + 2), generator=gen, device="cuda")
            part[:, D + 1] = part[:, D + 1].abs() + 0.5          # denominators
            if step == 2 and rank == 0:
                part[:4, D], part[:4, D + 1], part[:4, :D] = float("-inf"), 0.0, 0.0  # a rank that selected nothing
            want = merge_attention_partials(comm.all_gather(part), B, Hq, Sq, torch.bfloat16, sinks)
            got = ex.merge(part, torch.bfloat16, sinks)
            ok &= bool(torch.equal(got, want))
        ok &= ex.wait_errors() == 0
        # replayed by a CUDA graph: the step number advances on the device
        part = torch.randn((rows, D + 2), device="cuda")
        part[:, D + 1] = part[:, D + 1].abs() + 0.5
        want = merge_attention_partials(comm.all_gather(part), B, Hq, Sq, torch.bfloat16, None)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            ex.merge(part, torch.bfloat16, None)  # warm-up on the capture stream
            stream.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = ex.merge(part, torch.bfloat16, None)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        ok &= bool(torch.equal(out, want)) and ex.wait_errors() == 0
        results[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_gpu_peer_exchange_two_nccl_ranks():
    """`sah_attn_exchange_merge` on two GPUs against all-gather + `sah_attn_merge_parts`, bit for
    bit, eagerly and replayed by a CUDA graph.  Needs two GPUs (skipped on a one-GPU box)."""
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_nccl_rank, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: True, 1: True}
