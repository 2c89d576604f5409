"""MagicPig: SimHash (LSH) sampling of keys with collision-probability weights.

Reference: .../maskers/sampling/implementations/magic_pig.py (config :27-76,
bit packing :120-150, centring :152-183, caches :185-330, MIPS transform
:332-372, probabilities :374-403, matching :405-463, projections :465-508,
add_mask :510-593).

Keys and queries are centred by the per-head key mean, mapped to unit-norm
vectors by the Neyshabur-Srebro transform (keys scaled by the largest key norm of
the whole tensor and extended by sqrt(M^2 - |k|^2) / M, queries normalised and
extended by 0), and hashed by `lsh_l` tables of `lsh_k` random hyperplanes.  A key
is sampled when at least one of its table codes equals the query's; it then carries
the probability of that event, 1 - (1 - (1 - theta/pi)^k)^l, as its weight.

The reference materialises signatures as int64 `[B, Hq, S, L]` and probabilities for
every key.  Here the signatures of a layer live in a `PackedLSHSignatures`
(one code per table and key, key-major rows, once per KV head), a match kernel streams
them, and probabilities are evaluated for matched keys only.

In bfloat16 decode (at most four mask rows per KV group, previous mask empty or with unit
weights) the mask is returned with a `DeferredLSHWeights` payload: the matched set and what
the attention kernel needs to turn the K row it gathers anyway into the key's weight
(`sah_masked_attention_lsh`).  Nothing then reads the matched K rows a second time and no
weight array is written.  Whoever asks the mask for its indices, weights or dense form gets
them from the probability kernel, which rounds every step as the reference does
(`MagicPig.fused_weights = False` makes that the only path).

`sparse_meta_data` keys are the reference's: `"projections"[layer]` (`[D+1, L*K]`,
used as is when pre-populated), `"key_mean"[layer]` (`[B, Hq, 1, D]`, used as is when
pre-populated) and `"key_signature"[layer]` (the packed handle; a reference-layout
int64 tensor is converted on first use).
"""

import os
from dataclasses import dataclass, field
from typing import Any, Dict, Literal, Optional, Tuple

import torch

from ..... import _native_ops
from ....._native_ops import _native
from .....utils.kv_utils import _get_num_key_value_groups
from .....utils.mask import Mask, NativeBits, words_per_row
from ...base import MaskerConfig, MaskerRegistry
from ..base import SamplingMasker, SamplingMaskerConfig


@dataclass
class MagicPigConfig(SamplingMaskerConfig):
    """lsh_l tables of lsh_k bits; `center` subtracts the key mean first; `packing` only
    names the reference's signature storage ("int64" or "float32" give the same matches);
    `seed` (+ layer index) seeds the projections."""

    lsh_l: int
    lsh_k: int
    center: bool = True
    packing: Literal["int64", "float32"] = "int64"
    seed: Optional[int] = 42
    search_space: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.lsh_l <= 0:
            raise ValueError(f"lsh_l must be positive, got {self.lsh_l}")
        if self.lsh_k <= 0:
            raise ValueError(f"lsh_k must be positive, got {self.lsh_k}")
        if self.packing not in ["int64", "float32"]:
            raise ValueError(f"packing must be 'int64' or 'float32', got {self.packing}")
        if self.packing == "int64" and self.lsh_k > 64:
            raise ValueError(f"For 'int64' packing, lsh_k must be <= 64, but got {self.lsh_k}")
        if self.seed is None:
            raise ValueError("seed cannot be None")


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class PackedLSHSignatures:
    """LSH state of one layer's keys.

    codes    uint8 (lsh_k <= 8) or int16 `[B, Hkv, capacity, pitch]`: the L table codes of key s
             in row s, zero-padded to `pitch` (L rounded up to a whole number of 16-byte chunks)
    norms    float32 `[B, Hkv, capacity]`: norm of the centred key (rounded to the key dtype)
    max_norm int32 `[1]`: float bits of the largest norm seen so far
    dens     float32 `[B, Hkv, capacity]`: norm of the transformed key + 1e-8 (a per-key constant
             of the probability formula), valid for the maximum norm in `dens_max`
    length   number of valid keys
    """

    def __init__(self, codes: torch.Tensor, norms: torch.Tensor, max_norm: torch.Tensor,
                 length: int, lsh_k: int, lsh_l: int) -> None:
        self.codes, self.norms, self.max_norm, self.length = codes, norms, max_norm, length
        self.lsh_k, self.lsh_l = lsh_k, lsh_l
        self.dens = torch.zeros_like(norms)
        self.dens_max = torch.zeros_like(max_norm)
        # sequence-sharded use: total key count at which max_norm was last reduced over the shards
        self.synced_total: Optional[int] = None

    @property
    def capacity(self) -> int:
        return self.codes.shape[2]

    @property
    def shape(self) -> Tuple[int, ...]:
        return (self.codes.shape[0], self.codes.shape[1], self.length, self.lsh_l)

    @staticmethod
    def pitch(lsh_l: int, lsh_k: int) -> int:
        per16 = 16 if lsh_k <= 8 else 8
        return _round_up(lsh_l, per16)

    @classmethod
    def allocate(cls, B: int, Hkv: int, L: int, lsh_k: int, n_keys: int, device) -> "PackedLSHSignatures":
        cap = _round_up(n_keys + max(256, n_keys // 8), 32)
        code_dtype = torch.uint8 if lsh_k <= 8 else torch.int16
        return cls(torch.zeros((B, Hkv, cap, cls.pitch(L, lsh_k)), dtype=code_dtype, device=device),
                   torch.zeros((B, Hkv, cap), dtype=torch.float32, device=device),
                   torch.zeros(1, dtype=torch.int32, device=device), 0, lsh_k, L)

    def grown(self, n_keys: int) -> "PackedLSHSignatures":
        if n_keys <= self.capacity:
            return self
        B, Hkv = self.codes.shape[:2]
        new = PackedLSHSignatures.allocate(B, Hkv, self.lsh_l, self.lsh_k, n_keys, self.codes.device)
        new.codes[:, :, : self.length] = self.codes[:, :, : self.length]
        new.norms[..., : self.length] = self.norms[..., : self.length]
        new.max_norm.copy_(self.max_norm)
        new.dens[..., : self.length] = self.dens[..., : self.length]
        new.dens_max.copy_(self.dens_max)
        new.length = self.length
        new.synced_total = self.synced_total
        return new

    def to_reference_layout(self, n_query_heads: int) -> torch.Tensor:
        """int64 `[B, Hq, length, L]`, the tensor the reference caches (magic_pig.py:120-150)."""
        G = n_query_heads // self.codes.shape[1]
        codes = self.codes[:, :, : self.length, : self.lsh_l].to(torch.int64)
        if self.codes.dtype == torch.int16:
            codes = codes & 0xFFFF
        return codes.repeat_interleave(G, dim=1).contiguous()

    @classmethod
    def from_reference_layout(cls, sig: torch.Tensor, n_kv_heads: int, lsh_k: int) -> "PackedLSHSignatures":
        """Adopt signatures cached by the reference (packed int64 `[B, Hq, S, L]`); the key
        norms are filled by the caller."""
        B, Hq, S, L = sig.shape
        G = Hq // n_kv_heads
        new = cls.allocate(B, n_kv_heads, L, lsh_k, S, sig.device)
        new.codes[:, :, :S, :L] = sig[:, ::G].to(new.codes.dtype)
        return new


class DeferredLSHWeights:
    """What `sah_attn_plan_lsh` + `sah_masked_attention_lsh` need of one MagicPig call, and the
    way back to an ordinary bitmap + weight array (`materialise`)."""

    def __init__(self, masker: "MagicPig", previous_mask: Mask, match_bits: torch.Tensor,
                 unit_bits: Optional[torch.Tensor], qhat: torch.Tensor, qmu: torch.Tensor,
                 qunit: torch.Tensor, sig: PackedLSHSignatures, table: torch.Tensor,
                 keys: torch.Tensor, mean: Optional[torch.Tensor], shape: Tuple[int, int, int, int],
                 G: int, weight_table: Optional[torch.Tensor] = None) -> None:
        self.masker, self.previous_mask = masker, previous_mask
        self.match_bits, self.unit_bits = match_bits, unit_bits
        self.qhat, self.qmu, self.qunit = qhat, qmu, qunit
        self.sig, self.table, self.keys, self.mean = sig, table, keys, mean
        self.weight_table = weight_table  # cosine -> 1 / (p + 1e-6), what the attention kernel reads
        self.shape, self.G = shape, G
        self.device = match_bits.device

    def materialise(self) -> NativeBits:
        """`previous.merge_mask(matches with their collision probabilities)`, every operation of
        the probability rounded as the reference rounds it (magic_pig.py:374-403, :581-593)."""
        B, Hq, Sq, S = self.shape
        rows = B * Hq * Sq
        this = NativeBits(self.match_bits, rows, S)
        self.masker._probabilities(this, self.keys, self.qunit, self.sig, self.mean, self.table,
                                   self.shape, self.G, self.previous_mask.dtype)
        merged = self.previous_mask.merge_mask(
            Mask._from_native(self.shape, self.previous_mask.dtype, this), inplace=False)
        return merged.native_bits()


@MaskerRegistry.register(MagicPigConfig)
class MagicPig(SamplingMasker):
    """LSH-sampled keys weighted by their collision probability."""

    #: bfloat16 decode: leave the weights to the attention kernel (see the module docstring)
    fused_weights: bool = True

    def __init__(self, config: MagicPigConfig) -> None:
        super().__init__(config)
        self.lsh_l = config.lsh_l
        self.lsh_k = config.lsh_k
        self.center = config.center
        self.packing = config.packing
        self.seed = config.seed

    # ------------------------------------------------------------------ caches
    def _validate_inputs(self, sparse_meta_data, kwargs: Dict[str, Any]) -> int:
        if sparse_meta_data is None:
            raise ValueError("sparse_meta_data cannot be None")
        layer_idx = kwargs.get("layer_idx")
        if layer_idx is None:
            raise ValueError("layer_idx must be provided in kwargs")
        return layer_idx

    def _projection(self, meta: Dict[Any, Any], layer_idx: int, keys: torch.Tensor) -> torch.Tensor:
        proj = meta.setdefault("projections", {}).get(layer_idx)
        if proj is None:
            generator = torch.Generator(device=keys.device)
            generator.manual_seed(self.seed + layer_idx)
            proj = torch.randn(keys.shape[-1] + 1, self.lsh_k * self.lsh_l, device=keys.device,
                               dtype=keys.dtype, generator=generator)
            meta["projections"][layer_idx] = proj
        if proj.device != keys.device or proj.dtype != keys.dtype or not proj.is_contiguous():
            proj = proj.to(device=keys.device, dtype=keys.dtype).contiguous()
        return proj

    def _key_mean(self, meta: Dict[Any, Any], layer_idx: int, keys: torch.Tensor, G: int,
                  lib, st, shard=None) -> Optional[torch.Tensor]:
        """Compact `[B, Hkv, D]` key mean in the key dtype (None when center=False); the
        reference-layout `[B, Hq, 1, D]` tensor is what sits in sparse_meta_data."""
        cache = meta.setdefault("key_mean", {})
        cache.setdefault(layer_idx, None)
        if not self.center:
            return None
        B, Hkv, S, D = keys.shape
        if cache[layer_idx] is None:
            sums = torch.zeros((B, Hkv, D), dtype=torch.float64, device=keys.device)
            _native.check(
                lib.sah_lsh_key_sums(keys.data_ptr(), _native.dtype_code(keys.dtype), keys.stride(0),
                                     keys.stride(1), keys.stride(2), B, Hkv, 0, S, D, sums.data_ptr(), st),
                "sah_lsh_key_sums")
            if shard is not None:  # the mean is over the whole sequence
                shard.comm.all_reduce_sum_(sums)
                S = shard.total
            mean = (sums / S).to(torch.float32).to(keys.dtype)
            cache[layer_idx] = mean.repeat_interleave(G, dim=1).unsqueeze(2)
        full = cache[layer_idx]
        compact = getattr(self, "_mean_compact", {}).get(layer_idx)
        if compact is None or compact[0] is not full:
            compact = (full, full[:, ::G, 0, :].to(device=keys.device, dtype=keys.dtype).contiguous())
            if not hasattr(self, "_mean_compact"):
                self._mean_compact = {}
            self._mean_compact[layer_idx] = compact
        return compact[1]

    def _update_key_signatures(self, meta: Dict[Any, Any], layer_idx: int, keys: torch.Tensor,
                               n_query_heads: int, mean: Optional[torch.Tensor], proj: torch.Tensor,
                               lib, st, shard=None) -> PackedLSHSignatures:
        cache = meta.setdefault("key_signature", {})
        handle = cache.get(layer_idx)
        B, Hkv, S, D = keys.shape
        code = _native.dtype_code(keys.dtype)
        sms = _native.sm_count(keys.device)
        kargs = (keys.data_ptr(), code, keys.stride(0), keys.stride(1), keys.stride(2), B, Hkv)

        def stats(h: PackedLSHSignatures, s0: int, s1: int) -> None:
            _native.check(lib.sah_lsh_key_stats(*kargs, s0, s1, D, _native.ptr(mean), h.capacity,
                                                h.norms.data_ptr(), h.max_norm.data_ptr(), sms, st),
                          "sah_lsh_key_stats")

        adopted = isinstance(handle, torch.Tensor)
        if adopted:  # cached by the reference implementation
            handle = PackedLSHSignatures.from_reference_layout(handle, Hkv, self.lsh_k)
            n_cached = cache[layer_idx].shape[2]
            if n_cached > S:
                raise ValueError(f"Current number of keys ({S}) is less than cached number of keys ({n_cached})")
            stats(handle, 0, n_cached)
            handle.length = n_cached
        if handle is None:
            handle = PackedLSHSignatures.allocate(B, Hkv, self.lsh_l, self.lsh_k, S, keys.device)
        if S < handle.length:
            raise ValueError(
                f"Current number of keys ({S}) is less than cached number of keys ({handle.length})")
        # With a sequence shard the maximum key norm is over all shards: whenever the total
        # length moved (any rank got new keys) every rank joins one 4-byte max-reduction.
        resync = shard is not None and handle.synced_total != shard.total
        if S > handle.length or resync:
            handle = handle.grown(S)
            s0 = handle.length
            stats(handle, s0, S)
            if resync:
                shard.comm.all_reduce_max_(handle.max_norm)
                handle.synced_total = shard.total
        s_new0 = handle.length
        if S > handle.length:
            s0 = handle.length
            done = False
            if self._tensor_core_build(keys, S - s0, D):
                done = self._sign_on_tensor_cores(lib, keys, s0, S, mean, handle, proj, sms, st)
            if not done:
                _native.check(
                    lib.sah_lsh_key_sign(*kargs, s0, S, D, _native.ptr(mean), handle.norms.data_ptr(),
                                         handle.max_norm.data_ptr(), proj.data_ptr(), self.lsh_l, self.lsh_k,
                                         handle.capacity, handle.codes.data_ptr(), st), "sah_lsh_key_sign")
            handle.length = S
        if S > s_new0 or resync or adopted:
            # per-key constants of the probability formula: the new keys, or every key when
            # the maximum norm moved (the kernel compares it with the one it last used)
            _native.check(
                lib.sah_lsh_key_den(*kargs, 0 if adopted else s_new0, S, D, _native.ptr(mean),
                                    handle.norms.data_ptr(), handle.capacity, handle.max_norm.data_ptr(),
                                    handle.dens_max.data_ptr(), handle.dens.data_ptr(), sms, st),
                "sah_lsh_key_den")
        cache[layer_idx] = handle
        return handle

    # Ranges of at least this many keys are hashed on the tensor cores (a decode step's single
    # appended key stays on the one-launch fixed-order kernel).
    tensor_core_build_min_keys = 4096

    def _tensor_core_build(self, keys: torch.Tensor, n_new: int, head_dim: int) -> bool:
        if os.environ.get("SAH_LSH_TC", "1") == "0":
            return False
        return (keys.dtype == torch.bfloat16 and head_dim == 128 and self.lsh_k == 8
                and n_new >= self.tensor_core_build_min_keys
                and keys.stride(3) == 1 and all((keys.stride(i) * 2) % 16 == 0 for i in range(3))
                and keys.data_ptr() % 16 == 0)

    def _sign_on_tensor_cores(self, lib, keys, s0, s1, mean, handle, proj, sms, st) -> bool:
        """Signatures of keys [s0, s1) by `sah_lsh_key_sign_tc` (tcgen05 projections + fixed-order
        redo of the near-zero ones).  Returns False -- after reading two status words, an index
        build may synchronise -- when the redo list overflowed or a wait inside the kernel ran
        out; the caller then hashes the range with the fixed-order kernel."""
        B, Hkv = keys.shape[0], keys.shape[1]
        nbytes = int(lib.sah_lsh_key_sign_tc_ws_bytes(B, Hkv, s1 - s0))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=keys.device)
        _native.check(
            lib.sah_lsh_key_sign_tc(keys.data_ptr(), keys.stride(0), keys.stride(1), keys.stride(2), B, Hkv,
                                    s0, s1, keys.shape[3], _native.ptr(mean), handle.norms.data_ptr(),
                                    handle.max_norm.data_ptr(), proj.data_ptr(), self.lsh_l, self.lsh_k,
                                    handle.capacity, handle.codes.data_ptr(), ws.data_ptr(), nbytes, sms, st),
            "sah_lsh_key_sign_tc")
        status = ws[:8].view(torch.int32).tolist()
        self.last_tensor_core_build = {"redone_groups": status[0], "keys": (s1 - s0) * B * Hkv}
        return status[1] == 0 and status[0] <= (nbytes - 16) // 16

    # ------------------------------------------------------------------ public
    def add_mask(self, keys, queries, values, attention_mask, scaling, dropout,
                 sparse_meta_data: Dict[Any, Any], previous_mask: Mask,
                 **kwargs: Dict[str, Any]) -> Mask:
        layer_idx = self._validate_inputs(sparse_meta_data, kwargs)
        if previous_mask.is_full_mask():
            return previous_mask
        B, Hq, Sq, D = queries.shape
        Hkv, S = keys.shape[1], keys.shape[2]
        G = _get_num_key_value_groups(queries, keys)
        _native.require_cuda(keys, "keys")
        _native.require_cuda(queries, "queries")
        lib = _native.load()
        dev = keys.device
        st = _native.stream_of(dev)
        dtype = queries.dtype
        code = _native.dtype_code(dtype)
        k = keys if keys.stride(-1) == 1 else keys.contiguous()
        q = queries if queries.stride(-1) == 1 else queries.contiguous()

        shard = kwargs.get("sequence_shard")  # keys are columns [begin, begin + S) of `total`
        mean = self._key_mean(sparse_meta_data, layer_idx, k, G, lib, st, shard)
        proj = self._projection(sparse_meta_data, layer_idx, k)
        sig = self._update_key_signatures(sparse_meta_data, layer_idx, k, Hq, mean, proj, lib, st, shard)

        rows = B * Hq * Sq
        W = words_per_row(S)
        # the attention kernel can evaluate the weights itself for bfloat16 decode shapes when
        # everything selected so far has weight 1
        prev_nb = None
        fused = self.fused_weights and dtype == torch.bfloat16 and D in (64, 128) and G <= 4
        if fused and not previous_mask.is_empty:
            prev_nb = _native_ops.unit_weight_bits(previous_mask)
            fused = prev_nb is not None
        qcodes = torch.empty((rows, self.lsh_l), dtype=sig.codes.dtype, device=dev)
        qunit = torch.empty((rows, D), dtype=torch.float32, device=dev)
        qhat = torch.empty((rows, D), dtype=dtype, device=dev) if fused else None
        qmu = torch.empty(rows, dtype=torch.float32, device=dev) if fused else None
        _native.check(
            lib.sah_lsh_query(q.data_ptr(), code, q.stride(0), q.stride(1), q.stride(2), B, Hq, Sq, G, D,
                              _native.ptr(mean), proj.data_ptr(), self.lsh_l, self.lsh_k,
                              qcodes.data_ptr(), qunit.data_ptr(), _native.ptr(qhat), _native.ptr(qmu),
                              st), "sah_lsh_query")
        bits = torch.empty((rows, W), dtype=torch.int32, device=dev)
        _native.check(
            lib.sah_lsh_match(sig.codes.data_ptr(), sig.capacity, qcodes.data_ptr(), B, Hq, Sq, G,
                              self.lsh_l, self.lsh_k, S, W, None, bits.data_ptr(), st),
            "sah_lsh_match")
        if W * 32 > (S + 31) // 32 * 32:
            bits[:, (S + 31) // 32:].zero_()  # padding words of the row stride
        table = _native_ops.lsh_prob_table(dev, self.lsh_k, self.lsh_l) if dtype == torch.bfloat16 else None
        shape = (B, Hq, Sq, S)
        if fused:
            payload = DeferredLSHWeights(self, previous_mask, bits,
                                         None if prev_nb is None else prev_nb.bits, qhat, qmu, qunit,
                                         sig, table, k, mean, shape, G,
                                         _native_ops.lsh_weight_table(dev, self.lsh_k, self.lsh_l))
            return Mask._from_native(shape, previous_mask.dtype,
                                     NativeBits(None, rows, S, deferred=payload))
        nb = NativeBits(bits, rows, S)
        self._probabilities(nb, k, qunit, sig, mean, table, shape, G, dtype)
        this_mask = Mask._from_native(shape, previous_mask.dtype, nb)
        return previous_mask.merge_mask(this_mask, inplace=False)

    def _probabilities(self, nb: NativeBits, k: torch.Tensor, qunit: torch.Tensor,
                       sig: PackedLSHSignatures, mean: Optional[torch.Tensor],
                       table: Optional[torch.Tensor], shape: Tuple[int, int, int, int], G: int,
                       dtype: torch.dtype) -> None:
        """Fill `nb.data` with the collision probability of every entry of `nb` (:374-403)."""
        B, Hq, Sq, S = shape
        lib = _native.load()
        dev = k.device
        st = _native.stream_of(dev)
        nb.ensure_scan()
        data = torch.empty(nb.rows * S, dtype=dtype, device=dev)  # worst case; nothing is read back
        _native.check(
            lib.sah_lsh_prob(k.data_ptr(), _native.dtype_code(dtype), k.stride(0), k.stride(1),
                             k.stride(2), B, Hq, Sq, G, k.shape[-1], _native.ptr(mean),
                             sig.norms.data_ptr(), sig.dens.data_ptr(), sig.capacity,
                             sig.max_norm.data_ptr(), qunit.data_ptr(), nb.bits.data_ptr(),
                             nb.wpre.data_ptr(), nb.ptr.data_ptr(), nb.words, self.lsh_k, self.lsh_l,
                             _native.ptr(table), data.data_ptr(), _native.sm_count(dev), st),
            "sah_lsh_prob")
        nb.data = data

    @classmethod
    def create_from_config(cls, config: MaskerConfig) -> "MagicPig":
        if not isinstance(config, MagicPigConfig):
            raise ValueError(f"Invalid config type: {type(config)}")
        return cls(config)
