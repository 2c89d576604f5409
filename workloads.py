"""Seeded synthetic decode workloads: Q/K/V and masker parameters.

The reference measures this path on random tensors only
(profile/profile_research_attention.py:68-127).  These generators produce the
shapes and value distributions of the benchmark configurations from a seed,
with numpy's Philox generator so that every machine gets identical values.
All arrays are float32; `to_dtype` rounds them to the compute dtype.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np


def _rng(seed: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, stream]))


def _normalise(x: np.ndarray) -> np.ndarray:
    return x / np.maximum(np.linalg.norm(x, axis=-1, keepdims=True), 1e-12)


@dataclass
class DecodeWorkload:
    """One decode step of one layer."""

    name: str
    dtype: str                      # "f32" or "bf16"
    q: np.ndarray                   # [B, Hq, Sq, D]
    k: np.ndarray                   # [B, Hkv, S, D]
    v: np.ndarray                   # [B, Hkv, S, D]
    scaling: float
    stack: List[Tuple[str, Dict[str, Any]]] = field(default_factory=list)

    @property
    def shape(self) -> Tuple[int, int, int, int, int, int]:
        B, Hq, Sq, D = self.q.shape
        return B, Hq, self.k.shape[1], Sq, self.k.shape[2], D


def qkv_iid_outliers(seed: int, B: int, Hq: int, Hkv: int, S: int, D: int, Sq: int = 1,
                     n_outlier: int = 4, outlier_scale: float = 8.0):
    """N(0,1) everywhere; `n_outlier` fixed key channels scaled up."""
    q = _rng(seed, 0).standard_normal((B, Hq, Sq, D), dtype=np.float32)
    k = _rng(seed, 1).standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = _rng(seed, 2).standard_normal((B, Hkv, S, D), dtype=np.float32)
    chans = _rng(seed, 3).choice(D, size=n_outlier, replace=False)
    k[..., chans] *= np.float32(outlier_scale)
    return q, k, v


def qkv_planted(seed: int, B: int, Hq: int, Hkv: int, S: int, D: int, Sq: int = 1,
                frac: float = 0.01, cosine: float = 0.6):
    """K, V ~ N(0,1); per KV group a direction u; `frac` of the group's keys are
    turned to cosine `cosine` with u; the group's queries point along u (plus a
    little per-head noise), so attention is peaked on the planted keys."""
    G = Hq // Hkv
    k = _rng(seed, 1).standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = _rng(seed, 2).standard_normal((B, Hkv, S, D), dtype=np.float32)
    u = _normalise(_rng(seed, 4).standard_normal((B, Hkv, 1, D), dtype=np.float32))
    n_plant = max(1, int(frac * S))
    pick = _rng(seed, 5)
    for b in range(B):
        for h in range(Hkv):
            idx = pick.choice(S, size=n_plant, replace=False)
            rows = k[b, h, idx]
            norms = np.linalg.norm(rows, axis=-1, keepdims=True)
            uu = u[b, h]
            perp = _normalise(rows - (rows @ uu.T) * uu)
            k[b, h, idx] = norms * (cosine * uu + np.sqrt(1.0 - cosine * cosine) * perp)
    noise = _rng(seed, 6).standard_normal((B, Hkv, G, Sq, D), dtype=np.float32)
    qd = _normalise(u[:, :, None, :, :] + 0.3 * _normalise(noise))
    q = (np.sqrt(D) * qd).reshape(B, Hq, Sq, D).astype(np.float32)
    return q, k, v


def qkv_clustered(seed: int, B: int, Hq: int, Hkv: int, S: int, D: int, Sq: int = 1,
                  n_clusters: int = 64, sigma: float = 0.3):
    """Keys and values drawn around `n_clusters` unit-variance Gaussian centres."""
    centres_k = _rng(seed, 7).standard_normal((B, Hkv, n_clusters, D), dtype=np.float32)
    centres_v = _rng(seed, 8).standard_normal((B, Hkv, n_clusters, D), dtype=np.float32)
    assign = _rng(seed, 9).integers(0, n_clusters, size=(B, Hkv, S))
    bi = np.arange(B)[:, None, None]
    hi = np.arange(Hkv)[None, :, None]
    k = centres_k[bi, hi, assign] + sigma * _rng(seed, 1).standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = centres_v[bi, hi, assign] + sigma * _rng(seed, 2).standard_normal((B, Hkv, S, D), dtype=np.float32)
    q = _rng(seed, 0).standard_normal((B, Hq, Sq, D), dtype=np.float32)
    return q, k.astype(np.float32), v.astype(np.float32)


def hat_weights(seed: int, n_heads: int, head_dim: int, hidden: int, bits: int,
                n_layers: int = 3) -> Dict[str, List[np.ndarray]]:
    """Random-init hash MLPs, query and key sides separate: weights N(0, 1/fan_in)
    as `[heads, in, out]`, zero biases `[heads, out]`."""
    dims = [head_dim] + [hidden] * (n_layers - 1) + [bits]
    out: Dict[str, List[np.ndarray]] = {"query_matrix": [], "query_bias": [],
                                        "key_matrix": [], "key_bias": []}
    for side, base in (("query", 20), ("key", 40)):
        for l in range(n_layers):
            w = _rng(seed, base + l).standard_normal((n_heads, dims[l], dims[l + 1]), dtype=np.float32)
            out[f"{side}_matrix"].append((w / np.sqrt(dims[l])).astype(np.float32))
            out[f"{side}_bias"].append(np.zeros((n_heads, dims[l + 1]), np.float32))
    return out


def to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to the compute dtype's grid (still stored as float32)."""
    if dtype == "f32":
        return np.asarray(x, np.float32)
    f = np.ascontiguousarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32).reshape(f.shape)


# ---------------------------------------------------------------------------
# The benchmark configurations (full size by default; `scale` shrinks S and B
# for parity tests).
# ---------------------------------------------------------------------------
def sink_local_fp32(seed: int = 0, B: int = 1, Hq: int = 32, Hkv: int = 8, S: int = 4096,
                    D: int = 128, sink: int = 128, window: int = 256, Sq: int = 1) -> DecodeWorkload:
    q, k, v = qkv_iid_outliers(seed, B, Hq, Hkv, S, D, Sq)
    return DecodeWorkload("sink_local_fp32", "f32", q, k, v, 1.0 / np.sqrt(D),
                          [("sink", {"sink_size": sink}), ("local", {"window_size": window})])


def hashattention_bf16(seed: int = 0, B: int = 8, Hq: int = 32, Hkv: int = 8, S: int = 32768,
                       D: int = 128, sink: int = 128, window: int = 512, heavy=0.05,
                       bits: int = 32, hidden: int = 128, layers: int = 3,
                       activation: str = "silu", Sq: int = 1) -> DecodeWorkload:
    q, k, v = qkv_planted(seed, B, Hq, Hkv, S, D, Sq)
    w = {n: [to_dtype(a, "bf16") for a in arrs]
         for n, arrs in hat_weights(seed, Hq, D, hidden, bits, layers).items()}
    return DecodeWorkload(
        "hashattention_bf16", "bf16", to_dtype(q, "bf16"), to_dtype(k, "bf16"), to_dtype(v, "bf16"),
        1.0 / np.sqrt(D),
        [("sink", {"sink_size": sink}), ("local", {"window_size": window}),
         ("hash_topk", {"heavy_size": heavy, "bits": bits, "hidden": hidden, "layers": layers,
                        "activation": activation, "weights": w})])


def oracle_topk(seed: int = 0, dtype: str = "bf16", B: int = 4, Hq: int = 32, Hkv: int = 8,
                S: int = 65536, D: int = 128, sink: int = 128, window: int = 512, heavy=0.02,
                Sq: int = 1) -> DecodeWorkload:
    q, k, v = qkv_clustered(seed, B, Hq, Hkv, S, D, Sq)
    return DecodeWorkload(
        "oracle_topk_" + dtype, dtype, to_dtype(q, dtype), to_dtype(k, dtype), to_dtype(v, dtype),
        1.0 / np.sqrt(D),
        [("sink", {"sink_size": sink}), ("local", {"window_size": window}),
         ("oracle_topk", {"heavy_size": heavy})])


def oracle_topp(seed: int = 0, dtype: str = "bf16", B: int = 4, Hq: int = 32, Hkv: int = 8,
                S: int = 65536, D: int = 128, sink: int = 128, window: int = 512, top_p: float = 0.9,
                Sq: int = 1) -> DecodeWorkload:
    """Sink + Local + oracle top-p on the clustered keys of `oracle_topk`."""
    wl = oracle_topk(seed, dtype, B, Hq, Hkv, S, D, sink, window, 0.02, Sq)
    wl.name = "oracle_topp_" + dtype
    wl.stack = wl.stack[:2] + [("oracle_topp", {"top_p": top_p})]
    return wl


def quest(seed: int = 0, dtype: str = "bf16", B: int = 8, Hq: int = 32, Hkv: int = 8, S: int = 32768,
          D: int = 128, sink: int = 128, window: int = 512, heavy=0.05, page_size: int = 64,
          Sq: int = 1) -> DecodeWorkload:
    """Sink + Local + Quest page top-k on clustered keys (the shape of the HashAttention workload)."""
    wl = oracle_topk(seed, dtype, B, Hq, Hkv, S, D, sink, window, 0.02, Sq)
    wl.name = "quest_" + dtype
    wl.stack = wl.stack[:2] + [("quest_topk", {"heavy_size": heavy, "page_size": page_size})]
    return wl


def oracle_adaptive(seed: int = 0, dtype: str = "bf16", B: int = 4, Hq: int = 32, Hkv: int = 8,
                    S: int = 65536, D: int = 128, sink: int = 128, window: int = 512, heavy=0.02,
                    base_rate=0.05, epsilon: float = 0.05, delta: float = 0.05,
                    Sq: int = 1) -> DecodeWorkload:
    """Sink + Local + oracle top-k + adaptive (epsilon, delta) sampling over the rest."""
    wl = oracle_topk(seed, dtype, B, Hq, Hkv, S, D, sink, window, heavy, Sq)
    wl.name = "oracle_adaptive_" + dtype
    wl.stack = wl.stack + [("adaptive_sampling", {
        "base_rate_sampling": base_rate, "epsilon": epsilon, "delta": delta,
        "init_offset": sink, "local_offset": window})]
    return wl


def pqcache(seed: int = 0, dtype: str = "bf16", B: int = 1, Hq: int = 32, Hkv: int = 8,
            S: int = 131072, D: int = 128, sink: int = 64, window: int = 256, heavy=2048,
            group_factor: int = 16, bits: int = 8, kmeans_iter: int = 10, Sq: int = 1,
            n_clusters: int = 256) -> DecodeWorkload:
    """Keys from a mixture of Gaussian clusters; Sink + Local + PQCache top-k."""
    q, k, v = qkv_clustered(seed, B, Hq, Hkv, S, D, Sq, n_clusters=n_clusters)
    return DecodeWorkload(
        "pqcache_" + dtype, dtype, to_dtype(q, dtype), to_dtype(k, dtype), to_dtype(v, dtype),
        1.0 / np.sqrt(D),
        [("sink", {"sink_size": sink}), ("local", {"window_size": window}),
         ("pq_topk", {"heavy_size": heavy, "pq_group_factor": group_factor, "pq_bits": bits,
                      "kmeans_iter": kmeans_iter, "init_offset": sink, "metric": "euclidean"})])


def magicpig(seed: int = 0, dtype: str = "bf16", B: int = 1, Hq: int = 32, Hkv: int = 8,
             S: int = 1048576, D: int = 128, sink: int = 64, window: int = 256, lsh_l: int = 75,
             lsh_k: int = 8, Sq: int = 1, n_clusters: int = 64) -> DecodeWorkload:
    """Clustered keys; Sink + Local + MagicPig.  The hyperplanes are part of the workload
    (`stack[-1][1]["projection"]`, `[D+1, lsh_l*lsh_k]` in the dtype) and are handed to every
    implementation through `sparse_meta_data["projections"]`."""
    q, k, v = qkv_clustered(seed, B, Hq, Hkv, S, D, Sq, n_clusters=n_clusters)
    proj = to_dtype(_rng(seed, 70).standard_normal((D + 1, lsh_l * lsh_k)).astype(np.float32), dtype)
    return DecodeWorkload(
        "magicpig_" + dtype, dtype, to_dtype(q, dtype), to_dtype(k, dtype), to_dtype(v, dtype),
        1.0 / np.sqrt(D),
        [("sink", {"sink_size": sink}), ("local", {"window_size": window}),
         ("magicpig", {"lsh_l": lsh_l, "lsh_k": lsh_k, "center": True, "projection": proj})])


def clustered_kv_range(seed: int, B: int, Hkv: int, begin: int, end: int, D: int, device,
                       dtype: str = "bf16", n_clusters: int = 64, sigma: float = 0.3,
                       chunk: int = 32768):
    """Keys and values [B, Hkv, end - begin, D] of a long clustered sequence, generated on
    `device` in chunks of `chunk` keys, each chunk from its own seed: any key range gives the
    same values whichever way the sequence is cut into ranges (sequence-sharded runs at
    different GPU counts see one workload).  Cluster centres come from `seed` alone."""
    import torch

    tdt = torch_dtype(dtype)
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1000003 + 17)
    centres_k = torch.randn((B, Hkv, n_clusters, D), generator=g, device=device)
    centres_v = torch.randn((B, Hkv, n_clusters, D), generator=g, device=device)
    k = torch.empty((B, Hkv, end - begin, D), dtype=tdt, device=device)
    v = torch.empty((B, Hkv, end - begin, D), dtype=tdt, device=device)
    bi = torch.arange(B, device=device)[:, None, None]
    hi = torch.arange(Hkv, device=device)[None, :, None]
    for c in range(begin // chunk, (end + chunk - 1) // chunk):
        g.manual_seed(seed * 1000003 + 1000 + c)
        assign = torch.randint(0, n_clusters, (B, Hkv, chunk), generator=g, device=device)
        kc = centres_k[bi, hi, assign] + sigma * torch.randn((B, Hkv, chunk, D), generator=g, device=device)
        vc = centres_v[bi, hi, assign] + sigma * torch.randn((B, Hkv, chunk, D), generator=g, device=device)
        lo, hi_ = max(begin, c * chunk), min(end, (c + 1) * chunk)
        k[:, :, lo - begin:hi_ - begin] = kc[:, :, lo - c * chunk:hi_ - c * chunk].to(tdt)
        v[:, :, lo - begin:hi_ - begin] = vc[:, :, lo - c * chunk:hi_ - c * chunk].to(tdt)
    return k, v


def pq_init_indices(seed: int, groups: int, n_keys: int, n_cent: int) -> np.ndarray:
    """Seeded k-means initialisation: per group the first `n_cent` entries of a permutation."""
    rng = _rng(seed, 60)
    return np.stack([rng.permutation(n_keys)[:n_cent] for _ in range(groups)]).astype(np.int64)


# ---------------------------------------------------------------------------
# Turning a workload into device tensors and masker configs
# ---------------------------------------------------------------------------
def torch_dtype(dtype: str):
    import torch

    return {"f32": torch.float32, "bf16": torch.bfloat16}[dtype]


def to_torch(x: np.ndarray, dtype: str, device):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device=device, dtype=torch_dtype(dtype))


def masker_configs(stack: List[Tuple[str, Dict[str, Any]]], dtype: str, device="cpu") -> list:
    """Config dataclasses of `sparse_attention_hub` for a stack description.  The package is
    whichever one `sparse_attention_hub` resolves to on sys.path: the B200 package, or the
    reference itself (same import paths, class names and fields) when a caller times that."""
    from sparse_attention_hub.sparse_attention.research_attention.maskers import fixed

    out = []
    for kind, prm in stack:
        if kind == "sink":
            out.append(fixed.SinkMaskerConfig(sink_size=prm["sink_size"]))
        elif kind == "local":
            out.append(fixed.LocalMaskerConfig(window_size=prm["window_size"]))
        elif kind == "oracle_topk":
            out.append(fixed.OracleTopKConfig(heavy_size=prm["heavy_size"]))
        elif kind == "oracle_topp":
            out.append(fixed.OracleTopPMaskerConfig(top_p=prm["top_p"]))
        elif kind == "quest_topk":
            from sparse_attention_hub.sparse_attention.research_attention.maskers.fixed import (
                implementations as fixed_impl)
            out.append(fixed_impl.QuestTopKMaskerConfig(heavy_size=prm["heavy_size"], page_size=prm["page_size"],
                                                   label_bits=prm.get("label_bits", 16)))
        elif kind == "hash_topk":
            w = {0: {name: [to_torch(a, dtype, device) for a in arrs]
                     for name, arrs in prm["weights"].items()}}
            out.append(fixed.HashAttentionTopKMaskerConfig(
                heavy_size=prm["heavy_size"], hat_bits=prm["bits"], hat_mlp_layers=prm["layers"],
                hat_mlp_hidden_size=prm["hidden"], hat_mlp_activation=prm["activation"],
                hat_weights=w))
        elif kind == "pq_topk":
            out.append(fixed.PQCacheConfig(
                heavy_size=prm["heavy_size"], pq_group_factor=prm["pq_group_factor"],
                pq_bits=prm["pq_bits"], kmeans_iter=prm["kmeans_iter"],
                init_offset=prm["init_offset"], metric=prm["metric"]))
        elif kind == "adaptive_sampling":
            from sparse_attention_hub.sparse_attention.research_attention.maskers.sampling import (
                implementations as sampling)
            out.append(sampling.AdaptiveSamplingMaskerConfig(
                base_rate_sampling=prm["base_rate_sampling"], epsilon=prm["epsilon"],
                delta=prm["delta"], init_offset=prm["init_offset"], local_offset=prm["local_offset"]))
        elif kind == "random_sampling":
            from sparse_attention_hub.sparse_attention.research_attention.maskers import sampling
            out.append(sampling.RandomSamplingMaskerConfig(sampling_rate=prm["sampling_rate"]))
        elif kind == "magicpig":
            from sparse_attention_hub.sparse_attention.research_attention.maskers import sampling
            out.append(sampling.MagicPigConfig(lsh_l=prm["lsh_l"], lsh_k=prm["lsh_k"],
                                               center=prm.get("center", True)))
        else:
            raise ValueError(f"unknown masker kind {kind}")
    return out


def research_attention(stack, dtype: str, device="cpu"):
    from sparse_attention_hub.sparse_attention.research_attention import (ResearchAttention,
                                                                          ResearchAttentionConfig)

    return ResearchAttention.create_from_config(
        ResearchAttentionConfig(masker_configs=masker_configs(stack, dtype, device)))
