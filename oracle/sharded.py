"""Sequence-sharded decode restated on numpy: one rank's part of a masker stack with the
positions and sizes of the whole sequence, the attention partial of its key range, and the
associative combine of the partials.  The collectives are whatever `comm` provides
(`all_reduce_sum`, `all_reduce_max`, `all_gather` on numpy arrays), so the same code runs
under torch.distributed (gloo) and in a single process.
"""

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from . import attention, hashattention, magicpig, mask_ops, topk
from .bf16 import round_to
from .stacks import StackState


class LocalComm:
    """world = 1."""

    rank, world = 0, 1

    def all_reduce_sum(self, x):
        return x

    def all_reduce_max(self, x):
        return x

    def all_gather(self, x):
        return np.asarray(x)[None]


class TorchComm:
    """numpy arrays through a torch.distributed process group."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self._dist, self.group = dist, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def _reduce(self, x, op):
        import torch

        t = torch.from_numpy(np.ascontiguousarray(x).copy())
        self._dist.all_reduce(t, op=op, group=self.group)
        return t.numpy()

    def all_reduce_sum(self, x):
        return self._reduce(x, self._dist.ReduceOp.SUM)

    def all_reduce_max(self, x):
        return self._reduce(x, self._dist.ReduceOp.MAX)

    def all_gather(self, x):
        import torch

        t = torch.from_numpy(np.ascontiguousarray(x).copy())
        out = [torch.empty_like(t) for _ in range(self.world)]
        self._dist.all_gather(out, t, group=self.group)
        return np.stack([o.numpy() for o in out])


@dataclass
class Shard:
    begin: int
    total: int
    comm: Any


def plan_shards(total: int, world: int, align: int = 32) -> List[Tuple[int, int]]:
    per = (total + world - 1) // world
    per = (per + align - 1) // align * align
    return [(min(total, r * per), min(total, r * per + per)) for r in range(world)]


def _global_topk_local_part(scores_loc, active_loc, k, shard: Shard):
    """Top-k over the whole row (ties to the lowest global column), this rank's part.
    Every rank's (score, active) rows are gathered padded to the longest range."""
    n = scores_loc.shape[-1]
    lens = shard.comm.all_gather(np.array([n], np.int64)).reshape(-1)
    width = int(lens.max())
    pad_s = np.full(scores_loc.shape[:-1] + (width,), -np.inf, np.float32)
    pad_a = np.ones(scores_loc.shape[:-1] + (width,), bool)  # padding counts as active = excluded
    pad_s[..., :n], pad_a[..., :n] = scores_loc, active_loc
    all_s, all_a = shard.comm.all_gather(pad_s), shard.comm.all_gather(pad_a)
    cat_s = np.concatenate([all_s[r][..., : lens[r]] for r in range(len(lens))], axis=-1)
    cat_a = np.concatenate([all_a[r][..., : lens[r]] for r in range(len(lens))], axis=-1)
    sel = topk.topk_inactive(cat_s, cat_a, k)
    off = int(lens[: shard.comm.rank].sum())
    return sel[..., off:off + n]


def build_local_mask(stack, q, k_loc, dtype: str, shard: Shard, meta: Dict[str, Any]):
    """(dense local mask or None, full flag, empty flag)."""
    B, Hq, Sq, _ = q.shape
    n = k_loc.shape[2]
    st = StackState((B, Hq, Sq, n), dtype)
    cols = shard.begin + np.arange(n)  # global columns of the local keys
    for kind, prm in stack:
        if st.full:
            break
        if kind == "sink":
            size = mask_ops.effective_size(prm["sink_size"], shard.total)
            if shard.total <= size:
                st.full = True
                continue
            out = st.mask.copy()
            out[..., cols < size] = 1.0
            st.set(out)
        elif kind == "local":
            w = mask_ops.effective_size(prm["window_size"], shard.total)
            if shard.total <= w + Sq:
                st.full = True
                continue
            off = cols[None, :] - np.arange(Sq)[:, None]
            lo, hi = shard.total - Sq - w + 1, shard.total - Sq + 1
            out = st.mask.copy()
            out[..., (off >= lo) & (off < hi)] = 1.0
            out[..., off >= hi] = 0.0
            st.set(out)
        elif kind == "hash_topk":
            kk = mask_ops.effective_size(prm["heavy_size"], shard.total)
            if shard.total <= kk:
                st.full = True
                continue
            G = Hq // k_loc.shape[1]
            w = prm["weights"]
            kc = hashattention.signatures(attention.repeat_kv(k_loc, G), w["key_matrix"], w["key_bias"],
                                          prm["activation"], dtype)
            qc = hashattention.signatures(q, w["query_matrix"], w["query_bias"], prm["activation"], dtype)
            s = hashattention.scores(qc, kc, prm["bits"], dtype, None)
            sel = _global_topk_local_part(s, st.mask != 0, kk, shard)
            st.set(mask_ops.merge(st.mask, sel.astype(np.float32), dtype))
        elif kind == "oracle_topk":
            from . import qk
            kk = mask_ops.effective_size(prm["heavy_size"], shard.total)
            if shard.total <= kk:
                st.full = True
                continue
            s = qk.qk_scores(q, k_loc, dtype, None)
            sel = _global_topk_local_part(s, st.mask != 0, kk, shard)
            out = st.mask.copy()
            out[sel] = 1.0
            st.set(out)
        elif kind == "magicpig":
            magicpig.apply(prm, st, q, k_loc, meta, shard)
        else:
            raise ValueError(f"masker kind {kind} has no sequence-sharded restatement")
    return (None if (st.full or st.empty) else st.mask), st.full, st.empty


def merge_partials(num, den, mx, dtype: str, sinks=None):
    """num [G,B,Hq,Sq,D], den / mx [G,B,Hq,Sq,1] -> out [B,Sq,Hq,D] in `dtype`."""
    M = mx.max(axis=0)
    sc = np.exp(mx - M[None])
    n, d = (num * sc).sum(axis=0), (den * sc).sum(axis=0)
    if sinks is not None:
        s = np.asarray(sinks, np.float32).reshape(1, -1, 1, 1)
        new_max = np.maximum(M, s)
        scale = np.exp(M - new_max)
        n, d = n * scale, d * scale + np.exp(s - new_max)
    out = round_to((n / d).astype(np.float32), dtype)
    return np.ascontiguousarray(out.transpose(0, 2, 1, 3))


def run_sharded(stack, q, k_loc, v_loc, scaling: float, dtype: str, shard: Shard,
                meta: Optional[Dict[str, Any]] = None, sinks=None):
    """One rank's step: (local dense mask or None, full output [B,Sq,Hq,D], meta)."""
    meta = {} if meta is None else meta
    mask, full, empty = build_local_mask(stack, q, k_loc, dtype, shard, meta)
    num, den, mx = attention.masked_attention(q, k_loc, v_loc, mask, scaling, dtype,
                                              no_mask=mask is None, return_partials=True)
    out = merge_partials(shard.comm.all_gather(num), shard.comm.all_gather(den),
                         shard.comm.all_gather(mx), dtype, sinks)
    return mask, out, meta
