"""Sequence-sharded decode: one contiguous range of the KV cache per GPU.

Every per-key quantity of the masker stack (K, V, hash codes, LSH signatures) is independent
along the sequence, and softmax partials combine associatively, so a long context is split
into contiguous key ranges, one per rank.  Each rank runs the masker stack on its own range
with the positions and sizes of the whole sequence (`sequence_shard` reaches every masker
through `add_mask`'s keyword arguments), computes the unnormalised attention partial of its
range, and one all-gather of `(accumulator, running max, denominator)` per row followed by
`sah_attn_merge_parts` gives every rank the full output.  Build-time quantities that are
global in the reference -- MagicPig's key mean and maximum key norm
(maskers/sampling/implementations/magic_pig.py:175-176, :352-353) -- are reduced across the
ranks when keys arrive, not per step.

On NCCL ranks the all-gather and the merge are one kernel over peer memory instead
(`PeerExchange`, `sah_attn_exchange_merge`): every rank stores its partial straight into its
peers' receive buffers over NVLink, signals, and merges what arrived.

Collectives go through a small `ShardComm` interface: `DistComm` is `torch.distributed`
(NCCL on GPUs), `ThreadComm` runs the ranks as threads of one process (tests on one device).
Maskers that have not been taught about shards refuse a `sequence_shard` instead of
silently treating the local range as the whole sequence.
"""

from __future__ import annotations

import ctypes
import os
import threading
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ... import _native
from ..utils.mask_attention_utils import merge_attention_partials, native_masked_attention


class ShardComm:
    """The three collectives the sharded path needs."""

    rank: int = 0
    world: int = 1

    def all_reduce_sum_(self, t: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def all_reduce_max_(self, t: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """`[world, *t.shape]`, rank order."""
        raise NotImplementedError


class DistComm(ShardComm):
    """`torch.distributed` process group (NCCL for CUDA tensors, gloo for CPU tensors)."""

    def __init__(self, group=None) -> None:
        import torch.distributed as dist

        self._dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def all_reduce_sum_(self, t):
        self._dist.all_reduce(t, op=self._dist.ReduceOp.SUM, group=self.group)
        return t

    def all_reduce_max_(self, t):
        self._dist.all_reduce(t, op=self._dist.ReduceOp.MAX, group=self.group)
        return t

    def all_gather(self, t):
        t = t.contiguous()
        flat = t.reshape(-1)
        out = torch.empty(self.world * flat.numel(), dtype=t.dtype, device=t.device)
        self._dist.all_gather_into_tensor(out, flat, group=self.group)
        return out.view((self.world,) + tuple(t.shape))


class PeerExchange:
    """Receive buffer, flags and step counters of `sah_attn_exchange_merge` for one problem shape.

    The buffer and the flags live in one symmetric-memory allocation
    (`torch.distributed._symmetric_memory`), which maps every rank's copy into every process;
    the kernel then needs nothing but the peers' base addresses.  One rank per GPU: the
    kernels of different ranks wait on one another (bounded), so they must not share a device.
    Collective: every rank of the group constructs it, with the same shape, at the same point.
    """

    def __init__(self, comm: "DistComm", batch: int, heads: int, seq_len_queries: int, head_dim: int,
                 device: torch.device) -> None:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        lib = _native.load()
        self.shape = (batch, heads, seq_len_queries, head_dim)
        self.rank, self.world = comm.rank, comm.world
        rows = batch * heads * seq_len_queries
        nbytes = int(lib.sah_attn_exchange_bytes(self.world, batch, heads, seq_len_queries, head_dim))
        if nbytes <= 0 or self.world > 16:
            raise ValueError("PeerExchange: unsupported shape or more than 16 ranks")
        words = nbytes // 4 + self.world * rows
        group = comm.group if comm.group is not None else dist.group.WORLD
        self._mem = symm.empty(words, dtype=torch.float32, device=device)
        self._mem.zero_()
        self._handle = symm.rendezvous(self._mem, group)
        ptrs = [int(p) for p in self._handle.buffer_ptrs]
        self._bufs = (ctypes.c_void_p * self.world)(*ptrs)
        self._flags = (ctypes.c_void_p * self.world)(*[p + nbytes for p in ptrs])
        self.steps = torch.zeros(rows, dtype=torch.int32, device=device)
        self.errflag = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.current_stream(device).synchronize()
        dist.barrier(group=group)  # every buffer is zeroed before any peer stores into it

    def merge(self, part: torch.Tensor, dtype: torch.dtype, sinks: Optional[torch.Tensor]) -> torch.Tensor:
        """`part` [rows, D + 2] of this rank -> output [B, Sq, Hq, D] over all ranks."""
        B, Hq, Sq, D = self.shape
        lib = _native.load()
        part = part.contiguous()
        out = torch.empty((B, Sq, Hq, D), dtype=dtype, device=part.device)
        sk = None if sinks is None else sinks.to(device=part.device, dtype=torch.float32).contiguous()
        _native.check(
            lib.sah_attn_exchange_merge(part.data_ptr(), self._bufs, self._flags, self.rank, self.world, B, Hq,
                                        Sq, D, None if sk is None else sk.data_ptr(), _native.dtype_code(dtype),
                                        self.steps.data_ptr(), self.errflag.data_ptr(), out.data_ptr(),
                                        _native.stream_of(part.device)),
            "sah_attn_exchange_merge")
        return out

    def wait_errors(self) -> int:
        """Non-zero when a bounded wait for a peer ran out since the last call (synchronises)."""
        v = int(self.errflag.item())
        self.errflag.zero_()
        return v


def peer_exchange_allowed(comm: ShardComm, tensor: torch.Tensor) -> bool:
    """The peer-memory exchange needs NCCL ranks on distinct GPUs; `SAH_PEER_EXCHANGE=0` in the
    environment keeps the all-gather path."""
    if os.environ.get("SAH_PEER_EXCHANGE", "1") == "0":
        return False
    return isinstance(comm, DistComm) and comm.world > 1 and comm.world <= 16 and tensor.is_cuda


class ThreadComm(ShardComm):
    """Ranks are threads of one process; tensors meet in a shared slot list between two
    barriers.  Only host threads wait on each other: kernels never do."""

    def __init__(self, rank: int, world: int, slots: List[Any], barrier: threading.Barrier) -> None:
        self.rank, self.world, self._slots, self._barrier = rank, world, slots, barrier

    @classmethod
    def create(cls, world: int) -> List["ThreadComm"]:
        slots: List[Any] = [None] * world
        barrier = threading.Barrier(world)
        return [cls(r, world, slots, barrier) for r in range(world)]

    def _exchange(self, t: torch.Tensor) -> torch.Tensor:
        if t.is_cuda:
            # the other threads read this tensor from their own streams: finish producing it first
            torch.cuda.current_stream(t.device).synchronize()
        self._slots[self.rank] = t
        self._barrier.wait()
        stacked = torch.stack([s.to(t.device) for s in self._slots])
        if t.is_cuda:
            torch.cuda.current_stream(t.device).synchronize()  # done reading before anyone reuses
        self._barrier.wait()
        return stacked

    def all_reduce_sum_(self, t):
        return t.copy_(self._exchange(t.clone()).sum(dim=0))

    def all_reduce_max_(self, t):
        return t.copy_(self._exchange(t.clone()).amax(dim=0))

    def all_gather(self, t):
        return self._exchange(t.contiguous())


@dataclass
class SequenceShard:
    """The keys handed to a masker are columns `[begin, begin + keys.shape[2])` of `total`."""

    begin: int
    total: int
    comm: ShardComm


def plan_shards(total: int, world: int, align: int = 32) -> List[Tuple[int, int]]:
    """Contiguous `[begin, end)` ranges, one per rank: equal sizes rounded up to `align` keys
    (bitmap words stay whole), the last rank takes what is left (possibly nothing)."""
    if total < 0 or world <= 0:
        raise ValueError("total must be >= 0 and world > 0")
    per = (total + world - 1) // world
    per = (per + align - 1) // align * align
    out = []
    for r in range(world):
        b = min(total, r * per)
        out.append((b, min(total, b + per)))
    return out


class SequenceShardedAttention:
    """`ResearchAttention` over one rank's key range; `custom_attention` keeps the signature of
    `ResearchAttention.custom_attention` (research_attention/base.py:63-170) with local keys
    and values, and returns the full output on every rank."""

    def __init__(self, research_attention, comm: ShardComm, begin: int, total: int) -> None:
        self.research_attention = research_attention
        self.comm = comm
        self.begin = begin
        self.total = total
        self._exchange: Dict[Tuple[int, int, int, int], PeerExchange] = {}

    def keys_appended(self, n: int) -> None:
        """`n` keys joined the sequence (on the last rank); every rank calls this."""
        self.total += n

    def build_mask(self, queries, keys, values, attention_mask, scaling, dropout,
                   sparse_meta_data: Dict[Any, Any], **kwargs):
        shard = SequenceShard(self.begin, self.total, self.comm)
        if self.begin + keys.shape[2] > self.total:
            raise ValueError("local keys reach past the end of the sequence; call keys_appended() first")
        return self.research_attention.build_mask(queries, keys, values, attention_mask, scaling,
                                                  dropout, sparse_meta_data, sequence_shard=shard,
                                                  **kwargs)

    def custom_attention(self, module, queries: torch.Tensor, keys: torch.Tensor,
                         values: torch.Tensor, attention_mask: Optional[torch.Tensor],
                         scaling: float, dropout: float, **kwargs) -> Tuple[torch.Tensor, None]:
        if "sparse_meta_data" not in kwargs:
            raise ValueError(
                "sparse_meta_data must be provided in kwargs while calling custom_attention()")
        meta = kwargs.pop("sparse_meta_data")
        s_aux = kwargs.pop("s_aux", None)
        sinks = s_aux if isinstance(s_aux, torch.Tensor) else None
        B, Hq, Sq, D = queries.shape
        n_local = keys.shape[2]
        local_bias = None
        if attention_mask is not None:  # HF additive mask over the whole sequence
            local_bias = attention_mask[..., self.begin:self.begin + n_local]
        if n_local == 0:
            # every rank takes part in the maskers' reductions, so none may sit a step out
            raise ValueError("a rank of a sequence-sharded call must hold at least one key")
        mask = self.build_mask(queries, keys, values, local_bias, scaling, dropout, meta, **kwargs)
        _, part = native_masked_attention(queries, keys, values, local_bias, None, scaling,
                                          mask, return_partials=True)
        if peer_exchange_allowed(self.comm, part):
            shape = (B, Hq, Sq, D)
            ex = self._exchange.get(shape)
            if ex is None:  # collective; every rank meets the shape for the first time in the same call
                ex = self._exchange[shape] = PeerExchange(self.comm, B, Hq, Sq, D, part.device)
            return ex.merge(part, queries.dtype, sinks), None
        gathered = self.comm.all_gather(part)  # [world, rows, D + 2]
        out = merge_attention_partials(gathered, B, Hq, Sq, queries.dtype, sinks)
        return out, None
