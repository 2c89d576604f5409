"""PQCache: top-k by product-quantised key scores.

Reference: .../maskers/fixed/implementations/pq_top_k.py (config :24-60, add_mask
:77-150, k-means build :194-262, incremental quantisation :264-404, scoring
:406-490, mask :492-537) and utils/pq_utils.py (batched k-means :260-438).

Keys after `init_offset` are split into `pq_group_factor` sub-vectors; each
(batch, KV head, sub-vector) group has its own `2**pq_bits` centroids from batched
k-means.  A decode step builds one lookup table per query head (q_sub . centroid)
and streams the byte codes: score = sum of table entries, exact top-k over the
positions the previous mask leaves inactive, ties to the lowest key.

State in `sparse_meta_data` (per layer):
  "pq_centroids"  tensor [B, Hkv, n_sub, 2**bits, sub_d] in the key dtype (as the reference)
  "pq_codebook"   `PackedPQCodes` (bytes [B, Hkv, capacity, n_sub]); an int64 tensor
                  [B, n_keys, Hkv, n_sub] in the reference's layout is accepted and packed
k-means follows the reference's loop: assignment, centre update, empty clusters
reseeded from random keys, stop when every group's squared centre shift is below
1e-4 or after `kmeans_iter` iterations; the codes kept are those of the last
assignment, the centroids those after the last update.  Initial centres are the
first `2**bits` entries of a random permutation per group unless
`sparse_meta_data["pq_init_indices"][layer]` supplies them ([groups, 2**bits]).
"""

from dataclasses import dataclass
import os
from typing import Any, Dict, Optional, Tuple, Union

import torch

from ..... import _native_ops
from ....._native_ops import _native
from .....utils.mask import Mask
from ...base import AttentionTensorDimensions, MaskerConfig, MaskerRegistry
from ..base import TopKMasker, TopKMaskerConfig


@dataclass
class PQCacheConfig(TopKMaskerConfig):
    """heavy_size keys by PQ score; sub-vector dim = head_dim // pq_group_factor."""

    pq_group_factor: int
    pq_bits: int
    kmeans_iter: int
    init_offset: int
    metric: str

    def __post_init__(self) -> None:
        super().__post_init__()
        if self.pq_group_factor <= 0:
            raise ValueError(f"pq_group_factor must be > 0, got {self.pq_group_factor}")
        if self.pq_bits <= 0:
            raise ValueError(f"pq_bits must be > 0, got {self.pq_bits}")
        if self.kmeans_iter <= 0:
            raise ValueError(f"kmeans_iter must be > 0, got {self.kmeans_iter}")
        if self.init_offset < 0:
            raise ValueError(f"init_offset must be >= 0, got {self.init_offset}")
        if self.metric not in ["euclidean", "ip"]:
            raise ValueError(f"metric must be 'euclidean' or 'ip', got '{self.metric}'")


class PackedPQCodes:
    """Byte codes of one layer: uint8 `[B, Hkv, capacity, n_sub]`, `length` keys valid."""

    def __init__(self, codes: torch.Tensor, length: int) -> None:
        self.codes = codes
        self.length = length

    @property
    def shape(self) -> Tuple[int, ...]:
        """Shape in the reference's layout `[B, n_keys, Hkv, n_sub]`."""
        return (self.codes.shape[0], self.length, self.codes.shape[1], self.codes.shape[3])

    def to_reference_layout(self) -> torch.Tensor:
        return self.codes[:, :, : self.length].permute(0, 2, 1, 3).long()

    @classmethod
    def from_reference_layout(cls, codebook: torch.Tensor) -> "PackedPQCodes":
        n = codebook.shape[1]
        packed = torch.empty((codebook.shape[0], codebook.shape[2], _capacity_for(n), codebook.shape[3]),
                             dtype=torch.uint8, device=codebook.device)
        packed[:, :, :n] = codebook.permute(0, 2, 1, 3).to(torch.uint8)
        return cls(packed, n)


def _capacity_for(n_keys: int) -> int:
    return n_keys + max(256, n_keys // 16)


@MaskerRegistry.register(PQCacheConfig)
class PQCache(TopKMasker):
    """Product-quantised approximate top-k."""

    def __init__(self, config: PQCacheConfig) -> None:
        super().__init__(config)
        self.heavy_size = config.heavy_size
        self.pq_group_factor = config.pq_group_factor
        self.pq_bits = config.pq_bits
        self.kmeans_iter = config.kmeans_iter
        self.init_offset = config.init_offset
        self.metric = config.metric

    # ------------------------------------------------------------------ public
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        layer_idx = self._validate_inputs(sparse_meta_data, kwargs)
        if previous_mask.is_full_mask():
            return previous_mask
        dims = self._extract_tensor_dimensions(keys, queries)
        # On a sequence shard the keys at hand are one rank's range [begin, begin + n) of `total`
        # keys: sizes are those of the whole sequence, the quantised region starts at
        # init_offset of the whole sequence, the codebook is clustered over all ranks' keys, and
        # the top-k is taken over all ranks' scores.
        shard = kwargs.get("sequence_shard")
        total = shard.total if shard is not None else dims.seq_len_keys
        heavy = self._calculate_effective_size(self.heavy_size, total)
        if total <= heavy + self.init_offset + dims.seq_len_queries + 2 ** self.pq_bits:
            return self._create_full_mask(dims, previous_mask.dtype, previous_mask.device)
        if self.metric == "ip" and shard is not None:
            raise NotImplementedError("PQCache metric 'ip' on a sequence shard is not built")
        if self.pq_bits > 8:
            raise NotImplementedError("PQCache codes are bytes: pq_bits <= 8")
        _native.require_cuda(keys, "keys")
        self._initialize_pq_cache(sparse_meta_data, layer_idx)
        # first quantised key in local coordinates
        local_off = self.init_offset if shard is None else min(max(0, self.init_offset - shard.begin),
                                                               dims.seq_len_keys)
        if sparse_meta_data["pq_centroids"][layer_idx] is None:
            centroids, codes = self._perform_kmeans_clustering(keys, layer_idx, sparse_meta_data, local_off, shard)
        else:
            centroids, codes = self._handle_incremental_keys(keys, layer_idx, sparse_meta_data, local_off)
        scores = self._compute_pq_scores(queries, keys, centroids, codes, local_off)
        if shard is not None:
            if _native_ops.unit_weight_bits(previous_mask) is None:
                raise NotImplementedError("PQCache on a sequence shard needs a unit-weight previous mask")
            merged = _native_ops.topk_select_sharded(scores, previous_mask, heavy, shard.comm, local_off,
                                                     local_off + codes.length)
        else:
            merged = _native_ops.topk_select(scores, previous_mask, heavy, local_off, local_off + codes.length)
        shape = self._mask_shape(dims)
        if _native_ops.unit_weight_bits(previous_mask) is None:
            new_only = _native_ops.bits_andnot(merged, previous_mask.native_bits())
            return previous_mask.merge_mask(Mask._from_native(shape, previous_mask.dtype, new_only),
                                            inplace=False)
        return Mask._from_native(shape, previous_mask.dtype, merged)

    # --------------------------------------------------------------- internals
    def _validate_inputs(self, sparse_meta_data, kwargs: Dict[str, Any]) -> int:
        if sparse_meta_data is None:
            raise ValueError("sparse_meta_data cannot be None")
        layer_idx = kwargs.get("layer_idx")
        if layer_idx is None:
            raise ValueError("layer_idx must be provided in kwargs")
        return layer_idx

    def _should_use_full_attention(self, dims: AttentionTensorDimensions, heavy_size: int) -> bool:
        total_needed = heavy_size + self.init_offset + dims.seq_len_queries + 2 ** self.pq_bits
        return dims.seq_len_keys <= total_needed

    def _initialize_pq_cache(self, sparse_meta_data: Dict[str, Any], layer_idx: int) -> None:
        for name in ("pq_centroids", "pq_codebook", "pq_ip2l2_phi"):
            sparse_meta_data.setdefault(name, {}).setdefault(layer_idx, None)

    def _geometry(self, keys: torch.Tensor) -> Tuple[int, int, int, int, int]:
        B, Hkv, _, D = keys.shape
        n_sub = self.pq_group_factor
        return B, Hkv, n_sub, D // n_sub, 2 ** self.pq_bits

    def _key_args(self, keys: torch.Tensor):
        k = keys if keys.stride(-1) == 1 else keys.contiguous()
        return k, (k.data_ptr(), _native.dtype_code(k.dtype), k.stride(0), k.stride(1), k.stride(2))

    def _gather_subvectors(self, k: torch.Tensor, idx: torch.Tensor, local_off: int, shard) -> torch.Tensor:
        """Sub-vectors `[B, Hkv, n_sub, n_pick, sub_d]` (float32) of the quantised keys with the
        region-relative indices `idx` `[B, Hkv, n_sub, n_pick]`.  On a shard an index may name a
        key of another rank: every rank fills in what it owns and the ranks add up (one
        non-zero term per element, so the sum is exact)."""
        B, Hkv, n_local, D = k.shape
        n_sub = idx.shape[2]
        sub_d = D // n_sub
        dev = k.device
        if shard is None:
            pos, own = idx + local_off, None
        else:
            pos = idx + (self.init_offset - shard.begin)  # local key position of region index
            own = (pos >= local_off) & (pos < n_local)
            pos = pos.clamp(0, max(n_local - 1, 0))
        bi = torch.arange(B, device=dev).view(B, 1, 1, 1)
        hi = torch.arange(Hkv, device=dev).view(1, Hkv, 1, 1)
        si = torch.arange(n_sub, device=dev).view(1, 1, n_sub, 1)
        if n_local == 0:
            picked = torch.zeros((B, Hkv, n_sub, idx.shape[3], sub_d), dtype=torch.float32, device=dev)
        else:
            picked = k.reshape(B, Hkv, n_local, n_sub, sub_d)[bi, hi, pos, si].float()
        if own is not None:
            picked = torch.where(own.unsqueeze(-1), picked, torch.zeros_like(picked))
            shard.comm.all_reduce_sum_(picked)
        return picked

    def _perform_kmeans_clustering(self, keys: torch.Tensor, layer_idx: int,
                                   sparse_meta_data: Dict[str, Any], local_off: Optional[int] = None,
                                   shard=None):
        lib = _native.load()
        B, Hkv, n_sub, sub_d, n_cent = self._geometry(keys)
        local_off = self.init_offset if local_off is None else local_off
        n_local = keys.shape[2] - local_off                       # quantised keys on this rank
        n_keys = (shard.total if shard is not None else keys.shape[2]) - self.init_offset  # ... in all
        dev = keys.device
        st = _native.stream_of(dev)
        groups = B * Hkv * n_sub
        k, kargs = self._key_args(keys)
        if self.metric == "ip":
            # inner product -> L2 (utils/pq_utils.py:585-612): every sub-vector of the clustered keys
            # gets the column sqrt(phi - |x|^2), phi the largest |x|^2 of its group; the clustering
            # then runs on sub-vectors of sub_d + 1 channels of a tensor of its own
            sub = k[:, :, local_off:, :].reshape(B, Hkv, n_local, n_sub, sub_d)
            norms_sq = (sub ** 2).sum(dim=4, keepdim=True)
            phi = norms_sq.amax(dim=2, keepdim=True)                       # [B, Hkv, 1, n_sub, 1]
            k = torch.cat([sub, torch.sqrt(phi - norms_sq)], dim=4).reshape(B, Hkv, n_local, n_sub * (sub_d + 1))
            k = k.contiguous()
            kargs = (k.data_ptr(), _native.dtype_code(k.dtype), k.stride(0), k.stride(1), k.stride(2))
            sparse_meta_data["pq_ip2l2_phi"][layer_idx] = phi.permute(0, 1, 3, 2, 4).reshape(groups, 1, 1)
            sub_d += 1
            local_off = 0
        init = sparse_meta_data.get("pq_init_indices", {}).get(layer_idx)
        if init is None:
            init = torch.stack([torch.randperm(n_keys, device=dev)[:n_cent] for _ in range(groups)])
            if shard is not None:  # rank 0's draw for everybody
                init = shard.comm.all_reduce_sum_(init if shard.comm.rank == 0 else torch.zeros_like(init))
        init = init.to(device=dev, dtype=torch.long).reshape(B, Hkv, n_sub, n_cent)
        # initial centres: the chosen keys' sub-vectors, as float32 [groups][n_cent][sub_d]
        centroids = self._gather_subvectors(k, init, local_off, shard).reshape(groups, n_cent, sub_d).contiguous()
        codes = torch.empty((B, Hkv, _capacity_for(max(n_local, 1)), n_sub), dtype=torch.uint8, device=dev)
        cap = codes.shape[2]
        sums = torch.empty((groups, n_cent, sub_d), dtype=torch.float64, device=dev)
        counts = torch.empty((groups, n_cent), dtype=torch.int32, device=dev)
        shift2 = torch.empty(groups, dtype=torch.float32, device=dev)
        reseed_src = sparse_meta_data.get("pq_reseed_indices", {}).get(layer_idx)
        own_pos = torch.arange(n_cent, device=dev, dtype=torch.long).repeat(groups, 1).contiguous()
        # the distance contraction of the assignment runs on the tensor cores when the shapes
        # allow (bfloat16 keys, 8 channels per sub-vector, 16..256 centroids in multiples of 16)
        use_tc = (os.environ.get("SAH_PQ_TC", "1") != "0" and k.dtype == torch.bfloat16 and sub_d == 8
                  and 16 <= n_cent <= 256 and n_cent % 16 == 0 and k.data_ptr() % 16 == 0
                  and all((k.stride(i) * 2) % 16 == 0 for i in range(3)))
        tc_err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.last_build_used_tensor_cores = use_tc
        for it in range(self.kmeans_iter):
            if n_local > 0:
                if use_tc:
                    _native.check(lib.sah_pq_assign_tc(k.data_ptr(), k.stride(0), k.stride(1), k.stride(2), B, Hkv,
                                                       local_off, k.shape[2], local_off, n_sub, sub_d, n_cent,
                                                       centroids.data_ptr(), codes.data_ptr(), cap,
                                                       tc_err.data_ptr(), _native.sm_count(dev), st),
                                  "sah_pq_assign_tc")
                    if int(tc_err.item()) != 0:  # a bounded wait inside the kernel ran out: fixed-order kernel
                        use_tc = False
                        tc_err.zero_()
                if not use_tc:
                    _native.check(lib.sah_pq_assign(*kargs, B, Hkv, local_off, k.shape[2], local_off, n_sub,
                                                    sub_d, n_cent, centroids.data_ptr(), codes.data_ptr(), cap, 0,
                                                    st), "sah_pq_assign")
            sums.zero_()
            counts.zero_()
            if n_local > 0:
                _native.check(lib.sah_pq_accumulate(*kargs, B, Hkv, n_local, local_off, n_sub, sub_d, n_cent,
                                                    codes.data_ptr(), cap, sums.data_ptr(), counts.data_ptr(),
                                                    st), "sah_pq_accumulate")
            if reseed_src is not None:
                reseed = reseed_src[it].to(device=dev, dtype=torch.long).contiguous()
            else:
                reseed = torch.randint(0, n_keys, (groups, n_cent), device=dev)
                if shard is not None:
                    reseed = shard.comm.all_reduce_sum_(reseed if shard.comm.rank == 0
                                                        else torch.zeros_like(reseed))
            if shard is None:
                _native.check(lib.sah_pq_update(*kargs, B, Hkv, local_off, n_sub, sub_d, n_cent,
                                                sums.data_ptr(), counts.data_ptr(), reseed.data_ptr(),
                                                centroids.data_ptr(), shift2.data_ptr(), st),
                              "sah_pq_update")
            else:
                # sums of bfloat16 / float32 key values in float64 and counts add up exactly over
                # the ranks; the keys that re-seed empty clusters may live anywhere, so they are
                # gathered into a [B, Hkv, n_cent, D] table that the update kernel reads instead
                shard.comm.all_reduce_sum_(sums)
                shard.comm.all_reduce_sum_(counts)
                picked = self._gather_subvectors(k, reseed.reshape(B, Hkv, n_sub, n_cent), local_off, shard)
                table = picked.permute(0, 1, 3, 2, 4).reshape(B, Hkv, n_cent, n_sub * sub_d).to(k.dtype).contiguous()
                _native.check(lib.sah_pq_update(table.data_ptr(), _native.dtype_code(table.dtype), table.stride(0),
                                                table.stride(1), table.stride(2), B, Hkv, 0, n_sub, sub_d,
                                                n_cent, sums.data_ptr(), counts.data_ptr(), own_pos.data_ptr(),
                                                centroids.data_ptr(), shift2.data_ptr(), st), "sah_pq_update")
            if bool((shift2 < 1e-4).all().item()):  # the reference's convergence test (host sync)
                break
        cent_t = centroids.to(keys.dtype).reshape(B, Hkv, n_sub, n_cent, sub_d).contiguous()
        packed = PackedPQCodes(codes, max(n_local, 0))
        sparse_meta_data["pq_centroids"][layer_idx] = cent_t
        sparse_meta_data["pq_codebook"][layer_idx] = packed
        return cent_t, packed

    def _handle_incremental_keys(self, keys: torch.Tensor, layer_idx: int,
                                 sparse_meta_data: Dict[str, Any], local_off: Optional[int] = None):
        lib = _native.load()
        centroids: torch.Tensor = sparse_meta_data["pq_centroids"][layer_idx]
        cached = sparse_meta_data["pq_codebook"][layer_idx]
        B, Hkv, n_sub, sub_d, n_cent = self._geometry(keys)
        if isinstance(cached, torch.Tensor):
            cached = PackedPQCodes.from_reference_layout(cached)
        local_off = self.init_offset if local_off is None else local_off
        n_now = keys.shape[2] - local_off
        if cached is None:
            cached = PackedPQCodes(torch.empty((B, Hkv, _capacity_for(n_now), n_sub), dtype=torch.uint8,
                                               device=keys.device), 0)
        if n_now < cached.length:
            raise ValueError(f"Quantized region shrunk: {n_now} < {cached.length}")
        if n_now > cached.length:
            if n_now > cached.codes.shape[2]:
                grown = torch.empty((B, Hkv, _capacity_for(n_now), n_sub), dtype=torch.uint8,
                                    device=keys.device)
                grown[:, :, : cached.length] = cached.codes[:, :, : cached.length]
                cached.codes = grown
            k, kargs = self._key_args(keys)
            cd = centroids.shape[-1]  # sub_d, or sub_d + 1 when the codebook was clustered with metric "ip"
            cent32 = centroids.float().reshape(-1, n_cent, cd).contiguous()
            if cd == sub_d:
                _native.check(
                    lib.sah_pq_assign(*kargs, B, Hkv, local_off + cached.length, keys.shape[2],
                                      local_off, n_sub, sub_d, n_cent, cent32.data_ptr(),
                                      cached.codes.data_ptr(), cached.codes.shape[2], 1,
                                      _native.stream_of(keys.device)), "sah_pq_assign")
            else:
                # appended keys are augmented with a zero column (pq_top_k.py:371-383); the new rows
                # go through the same kernel as a tensor of their own, written behind the old codes
                first = local_off + cached.length
                new = k[:, :, first:, :].reshape(B, Hkv, n_now - cached.length, n_sub, sub_d)
                new = torch.cat([new, torch.zeros_like(new[..., :1])], dim=4)
                new = new.reshape(B, Hkv, n_now - cached.length, n_sub * cd).contiguous()
                _native.check(
                    lib.sah_pq_assign(new.data_ptr(), _native.dtype_code(new.dtype), new.stride(0), new.stride(1),
                                      new.stride(2), B, Hkv, 0, new.shape[2], -cached.length, n_sub, cd, n_cent,
                                      cent32.data_ptr(), cached.codes.data_ptr(), cached.codes.shape[2], 1,
                                      _native.stream_of(keys.device)), "sah_pq_assign")
            cached.length = n_now
        sparse_meta_data["pq_codebook"][layer_idx] = cached
        return centroids, cached

    def _compute_pq_scores(self, queries: torch.Tensor, keys: torch.Tensor, centroids: torch.Tensor,
                           codebook: PackedPQCodes, local_off: Optional[int] = None) -> torch.Tensor:
        """`[B, Hq, Sq, S]` scores; only columns of the clustered region are written."""
        lib = _native.load()
        B, Hq, Sq, D = queries.shape
        Hkv, S = keys.shape[1], keys.shape[2]
        n_sub, n_cent = centroids.shape[2], centroids.shape[3]
        sub_d = D // n_sub
        q = queries if queries.stride(-1) == 1 else queries.contiguous()
        cent = centroids[..., :sub_d].to(q.dtype).contiguous()
        scores = torch.empty((B, Hq, Sq, S), dtype=q.dtype, device=q.device)
        nbytes = int(lib.sah_pq_scores_ws_bytes(B, Hq, Hkv, Sq, n_sub, n_cent))
        tables = torch.empty(nbytes, dtype=torch.uint8, device=q.device)  # the query-centroid tables
        _native.check(
            lib.sah_pq_scores(q.data_ptr(), _native.dtype_code(q.dtype), q.stride(0), q.stride(1),
                              q.stride(2), cent.data_ptr(), codebook.codes.data_ptr(),
                              codebook.codes.shape[2], B, Hq, Hkv, Sq, codebook.length,
                              self.init_offset if local_off is None else local_off, S, n_sub, sub_d, n_cent,
                              scores.data_ptr(),
                              tables.data_ptr(), nbytes, _native.stream_of(q.device)), "sah_pq_scores")
        return scores

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "PQCache":
        if not isinstance(config, PQCacheConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
