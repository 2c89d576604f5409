"""Decode-time sparse attention benchmark: one layer, one decode step per "step".

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload: HashAttention top-k decode in bf16 -- batch 8, 32 query / 8 KV
heads, head_dim 128, 32768 keys, Sink(128) + Local(512) + HashAttention top-k at
5 % of keys, random-init 128->128->128->32 SiLU hash MLPs, queries planted on 1 %
of the keys.  A step is the steady-state decode call of one layer through the
public API (`ResearchAttention.custom_attention`): query hashing, Hamming top-k
over the cached packed key signatures, sink/local bands, plan, gather attention.
Key signatures are built once before timing (index build, reported separately).

Prints one JSON line (rank 0).  `value` is whole-job decode tokens per second
per layer with everything resident in HBM; `e2e` is the same through the public
API with host buffers: the step's query and newly appended key/value rows are
copied from pinned host memory, the appended key is hashed incrementally, and
the output is read back to the host, all inside the timed region.
With N > 1 every rank decodes its own batch on its own GPU (no data-path
collective; weak scaling) and the slowest rank's time is used.

`--impl reference` times the CPU restatement of the reference's algorithm
(oracle/, numpy) on the host cores on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
for p in (REPO, REPO / "sparse-attention-hub_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

METRIC = "sparse_decode_attn_tokens_per_s_per_layer"
UNIT = "tokens/s/layer"


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
def make_workload(name: str, seed: int, small: bool = False):
    from sparse_attention_hub import workloads

    if name == "hashattention":
        if small:
            return workloads.hashattention_bf16(seed=seed, B=2, S=4096)
        if os.environ.get("SAH_BENCH_BATCH"):  # profiler captures use a smaller batch
            return workloads.hashattention_bf16(seed=seed, B=int(os.environ["SAH_BENCH_BATCH"]))
        return workloads.hashattention_bf16(seed=seed)
    if name == "sink_local":
        return workloads.sink_local_fp32(seed=seed)
    if name == "oracle_topk":
        if small:
            return workloads.oracle_topk(seed=seed, B=1, S=8192)
        return workloads.oracle_topk(seed=seed)
    if name == "oracle_adaptive":
        if small:
            return workloads.oracle_adaptive(seed=seed, B=1, S=8192)
        return workloads.oracle_adaptive(seed=seed)
    if name == "oracle_topp":
        if small:
            return workloads.oracle_topp(seed=seed, B=1, S=8192)
        return workloads.oracle_topp(seed=seed)
    if name == "quest":
        if small:
            return workloads.quest(seed=seed, B=2, S=4096)
        return workloads.quest(seed=seed)
    if name == "pqcache":
        if small:
            return workloads.pqcache(seed=seed, S=16384, heavy=512, kmeans_iter=3)
        return workloads.pqcache(seed=seed)
    raise SystemExit(f"unknown workload {name}")


def workload_config(wl, name: str, extra: dict) -> dict:
    B, Hq, Hkv, Sq, S, D = wl.shape
    stack = []
    for kind, prm in wl.stack:
        stack.append({"masker": kind, **{k: v for k, v in prm.items() if k != "weights"}})
    cfg = {"workload": f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq={Sq} S={S} D={D} {wl.dtype}",
           "stack": stack, "seed_data": "synthetic, seeded (numpy Philox)"}
    cfg.update(extra)
    return cfg


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True) -> None:
        self.index = index
        self.enabled = enabled   # one sampler per job (rank 0) is enough
        self.proc = None
        self.lines: list = []
        self.first = 0           # lines before the timed region started
        self.thread = None

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "25", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment to enumerate the devices (seconds on an 8-GPU host):
            # the timed region starts once it delivers samples
            t0 = time.perf_counter()
            while not self.lines and time.perf_counter() - t0 < 15.0:
                time.sleep(0.02)
            self.first = len(self.lines)
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            # the region may be shorter than the sampling period: keep the GPU busy state
            # visible by waiting for at least one sample taken after it started
            t0 = time.perf_counter()
            while len(self.lines) < self.first + 2 and time.perf_counter() - t0 < 1.0:
                time.sleep(0.02)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            if len(self.lines) > self.first:
                self.lines = self.lines[self.first:]

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val == "Active":
                    reasons.add(nm)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)),
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# CPU baseline: the numpy restatement of the reference's algorithm
# ---------------------------------------------------------------------------
def cpu_baseline(wl, name: str, steps: int, warmup: int, budget_s: float = 25.0) -> dict:
    """Steady-state decode of one batch element on the host cores (dense in S, as the
    reference is); returns tokens/s/layer and what was sampled."""
    from oracle import attention as o_attn, hashattention as o_hash, stacks
    try:
        from threadpoolctl import threadpool_info
        blas_threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        blas_threads = os.cpu_count() or 1

    q, k, v = wl.q[:1], wl.k[:1], wl.v[:1]
    meta: dict = {}
    t_build0 = time.perf_counter()
    for kind, prm in wl.stack:
        if kind == "hash_topk":
            G = q.shape[1] // k.shape[1]
            w = prm["weights"]
            meta["hash_kcodes"] = o_hash.signatures_blas(o_attn.repeat_kv(k, G), w["key_matrix"],
                                                         w["key_bias"], prm["activation"], wl.dtype)
        if kind == "pq_topk":
            # The decode step's cost does not depend on how good the codebook is: centres are
            # the seeded initial keys (no Lloyd iteration), codes their nearest-centre assignment.
            from oracle import pq as o_pq
            from oracle.bf16 import round_to
            from sparse_attention_hub import workloads as wls
            off, n_sub, cent = prm["init_offset"], prm["pq_group_factor"], 2 ** prm["pq_bits"]
            X = o_pq.split_keys(k, off, n_sub)
            idx = wls.pq_init_indices(0, X.shape[0], X.shape[1], cent)
            C = X[np.arange(X.shape[0])[:, None], idx]
            codes = np.concatenate([o_pq.assign(X[g:g + 1], C[g:g + 1]) for g in range(X.shape[0])])
            Hkv_, n_ = k.shape[1], X.shape[1]
            meta["pq_centroids"] = round_to(C, wl.dtype).reshape(1, Hkv_, n_sub, cent, -1)
            meta["pq_codes"] = codes.reshape(1, Hkv_, n_sub, n_).transpose(0, 1, 3, 2)
        if kind == "adaptive_sampling":
            meta["adaptive_seed"] = 0
    t_build = time.perf_counter() - t_build0

    def step():
        return stacks.run_stack(wl.stack, q, k, v, wl.scaling, wl.dtype, meta=dict(meta))

    times = []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        step()
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_start > budget_s and len(times) >= 2:
            break
    per_step = float(np.median(times))
    return {"value": 1.0 / per_step, "unit": UNIT, "cores": int(blas_threads), "kind": "port",
            "sample": (f"batch element 0 of {name} (1 token/step), {len(times)} timed steps after "
                       f"{warmup} warm-up, median {per_step * 1e3:.1f} ms/step; numpy restatement of "
                       f"the reference algorithm (dense in S), BLAS matmuls on {blas_threads} threads, "
                       f"index build {t_build:.1f} s not included"),
            "ms_per_step": per_step * 1e3, "steps": len(times)}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload, args.seed, args.small)
    base = cpu_baseline(wl, args.workload, args.steps, args.warmup, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": base["steps"], "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": workload_config(wl, args.workload, {"sample": base["sample"]}),
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# native arm
# ---------------------------------------------------------------------------
def run_native(args) -> None:
    import torch

    from sparse_attention_hub import _native, workloads
    from sparse_attention_hub.sparse_attention.utils import mask_attention_utils as mau

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the native path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    _native.load()

    wl = make_workload(args.workload, args.seed + rank, args.small)
    B, Hq, Hkv, Sq, S, D = wl.shape
    tdt = workloads.torch_dtype(wl.dtype)
    esz = 2 if wl.dtype == "bf16" else 4
    ra = workloads.research_attention(wl.stack, wl.dtype, dev)
    q, k, v = (workloads.to_torch(a, wl.dtype, dev) for a in (wl.q, wl.k, wl.v))
    meta: dict = {}
    scaling = float(wl.scaling)

    def step(qq=q):
        return ra.custom_attention(None, qq, k, v, None, scaling, 0.0, sparse_meta_data=meta,
                                   layer_idx=0)[0]

    # index build (first call hashes every key); timed on its own
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = step()
    torch.cuda.synchronize()
    index_build_ms = (time.perf_counter() - t0) * 1e3

    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    # The decode step is captured once and replayed as a CUDA graph (public API:
    # sparse_attention_hub...research_attention.decode_graph.DecodeStepGraph).
    from sparse_attention_hub.sparse_attention.research_attention.decode_graph import DecodeStepGraph
    eager_step = step
    graph = None
    if not args.eager:
        graph = DecodeStepGraph(ra, q, k, v, None, scaling, meta, layer_idx=0)

        def step(qq=None):  # noqa: F811
            return graph.replay(qq)

    def timed_loop(n_steps: int):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(n_steps)]
        for a, b in evs:
            flush.zero_()
            a.record()
            step()
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # kernels of this library per step (a graph replay launches the same kernels
    # without passing through the library's host-side counter)
    launches0 = _native.launch_count()
    eager_step()
    launches_per_step = _native.launch_count() - launches0
    torch.cuda.synchronize()
    barrier()
    with ClockSampler(local_rank, enabled=(rank == 0)) as clocks:
        barrier()   # rank 0 may have waited for the sampler's first line
        per_step_ms = timed_loop(args.steps)
    barrier()
    launches = launches_per_step * args.steps
    total_ms = float(sum(per_step_ms))

    # kernel-level times: a separate eager pass, so that the timing events neither sit
    # inside `value` nor get baked into the graph
    graph_step = step
    step = eager_step
    eager_ms = float(sum(timed_loop(args.steps))) / args.steps
    _native.profile_enable(True)
    for slot in _native.PROFILE_SLOTS:
        _native.profile_read(slot)
    timed_loop(args.steps)
    prof = {slot: _native.profile_read(slot) for slot in _native.PROFILE_SLOTS}
    _native.profile_enable(False)
    step = graph_step

    # algorithmic bytes
    ucount = mau.last_union_counts()
    union_rows = int(ucount.sum().item()) if ucount is not None else 0
    row_bytes = 2 * D * esz
    attn_bytes = union_rows * row_bytes + (q.numel() + out.numel()) * esz
    stage_bytes = {"attention": attn_bytes}
    if any(kind == "hash_topk" for kind, _ in wl.stack):
        stage_bytes["hash_topk"] = B * Hq * S * 4
    if any(kind in ("oracle_topk", "oracle_topp") for kind, _ in wl.stack):
        stage_bytes["qk_scores"] = B * Hkv * S * D * esz
    for kind, prm in wl.stack:
        if kind == "pq_topk":  # one byte per sub-vector code per key and KV head
            stage_bytes["pq_scores"] = B * Hkv * (S - prm["init_offset"]) * prm["pq_group_factor"]
        if kind == "adaptive_sampling":  # the q.k scores of every row, read once
            stage_bytes["adaptive_budget"] = B * Hq * Sq * S * esz
        if kind == "oracle_topp":        # the same for the top-p threshold
            stage_bytes["topp_select"] = B * Hq * Sq * S * esz
        if kind == "quest_topk":         # per-page minimum and maximum of every channel, per KV head
            stage_bytes["quest_scores"] = B * Hkv * (-(-S // prm["page_size"])) * D * esz * 2
    step_bytes = sum(stage_bytes.values())

    # e2e: host buffers in, host result out, incremental key append
    q_host = torch.from_numpy(np.ascontiguousarray(wl.q)).to(tdt).pin_memory()
    kn_host = k[:, :, S - 1:S, :].cpu().pin_memory()
    vn_host = v[:, :, S - 1:S, :].cpu().pin_memory()
    out_host = torch.empty(out.shape, dtype=tdt).pin_memory()
    q_dev = torch.empty_like(q)
    key_cache = meta.get("key", {}).get(0)

    def mark_appended():
        if key_cache is not None:
            key_cache.length = S - 1  # the appended key is hashed inside the step

    e2e_graph = None
    if not args.eager:
        # same public call, captured with "one key appended since the last call"
        # the three host-to-device copies and the read-back are nodes of the same graph
        e2e_graph = DecodeStepGraph(ra, q, k, v, None, scaling, meta, layer_idx=0,
                                    before_each_call=mark_appended, host_query=q_host,
                                    host_inputs=[(k[:, :, S - 1:S, :], kn_host), (v[:, :, S - 1:S, :], vn_host)],
                                    host_output=out_host)

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            k[:, :, S - 1:S, :].copy_(kn_host, non_blocking=True)
            v[:, :, S - 1:S, :].copy_(vn_host, non_blocking=True)
            q_dev.copy_(q_host, non_blocking=True)
            mark_appended()
            o = eager_step(q_dev)
            out_host.copy_(o, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_times = []
    for _ in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        e2e_times.append(time.perf_counter() - t0)
    barrier()
    e2e_total = float(sum(e2e_times))

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([total_ms, e2e_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_total = float(t[0].item()), float(t[1].item())

    if rank == 0:
        peaks = {}
        peaks_file = REPO / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peaks = json.loads(peaks_file.read_text())
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
        ms_per_step = total_ms / args.steps
        tokens = B * world
        attn_ms, attn_n = prof["attention"]
        attn_avg_ms = attn_ms / max(attn_n, 1)
        achieved = attn_bytes / (attn_avg_ms * 1e-3) / 1e9 if attn_avg_ms > 0 else 0.0
        stage_times = {s: (ms / max(n, 1)) * 1e3 for s, (ms, n) in prof.items() if n > 0}
        # DRAM traffic of one attention launch: ncu (dram__bytes_read.sum + dram__bytes_write.sum)
        # measured 225 719 552 B for a launch of this workload whose algorithmic bytes were
        # 219 225 088 B (profiles/sections_decode_kernels_hashattention.md); traffic grows with
        # the rows gathered, so the launch timed here is scaled by that ratio.
        traffic, traffic_src = None, None
        if args.workload == "hashattention" and not args.small:
            traffic = attn_bytes * (225719552.0 / 219225088.0)
            traffic_src = ("ncu capture of one launch of this workload (read + write), scaled by "
                           "algorithmic bytes of the timed launch")
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_baseline(wl, args.workload, steps=10, warmup=2)
        line = {
            "metric": METRIC,
            "value": tokens / (ms_per_step * 1e-3),
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": wl.dtype,
            "data": "synthetic",
            "config": workload_config(wl, args.workload, {
                "parallelism": f"dp{world} (one batch per GPU, no data-path collective)",
                "l2": "flushed between steps (512 MiB memset outside the timed events)",
                "index_build_ms": index_build_ms,
                "launch": "eager" if args.eager else "CUDA graph replay of the public decode call",
                "eager_ms_per_step": eager_ms,
                "step_algorithmic_bytes": step_bytes,
                "step_hbm_fraction_of_measured_peak":
                    step_bytes / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
                "union_rows_per_step": union_rows,
                "kernel_us": stage_times,
            }),
            "roofline": {
                "kernel": "masked_attention_kernel (K/V row gather + weighted online softmax)",
                "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak if hbm_peak else None, "peak_source": peak_src,
                "frac_of_nominal_8TBs": achieved / 8000.0,
                "algorithmic_bytes_per_launch": attn_bytes,
                "avg_launch_us": attn_avg_ms * 1e3, "launches_timed": attn_n,
                "traffic": traffic, "traffic_source": traffic_src,
            },
            "e2e": {
                "value": tokens / (e2e_total / args.steps), "unit": UNIT,
                "h2d_bytes_per_step": int((q_host.numel() + kn_host.numel() + vn_host.numel()) * esz),
                "d2h_bytes_per_step": int(out_host.numel() * esz),
                "ms_per_step": e2e_total / args.steps * 1e3,
            },
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
        }
        if base is not None:
            line["cpu_baseline"] = {k_: base[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# long-context workloads: the KV cache is sequence-sharded over the GPUs (strong scaling)
# ---------------------------------------------------------------------------
LONG_WORKLOADS = {
    # name: (keys, small keys, stack builder)
    "magicpig": (1048576, 65536),
    "hashattention_long": (1048576, 65536),
}


def _long_stack(name: str, seed: int, Hq: int, D: int):
    from sparse_attention_hub import workloads

    if name == "magicpig":
        proj = workloads.to_dtype(
            workloads._rng(seed, 70).standard_normal((D + 1, 75 * 8)).astype(np.float32), "bf16")
        return [("sink", {"sink_size": 64}), ("local", {"window_size": 256}),
                ("magicpig", {"lsh_l": 75, "lsh_k": 8, "center": True, "projection": proj})]
    w = {n: [workloads.to_dtype(a, "bf16") for a in arrs]
         for n, arrs in workloads.hat_weights(seed, Hq, D, 128, 32, 3).items()}
    return [("sink", {"sink_size": 128}), ("local", {"window_size": 512}),
            ("hash_topk", {"heavy_size": 0.02, "bits": 32, "hidden": 128, "layers": 3,
                           "activation": "silu", "weights": w})]


def long_cpu_baseline(name: str, seed: int, S: int, budget_s: float = 25.0) -> dict:
    """The numpy restatement on a slice of the sequence (it is dense in the key count, so
    its time scales linearly with it); tokens/s/layer extrapolated to all S keys."""
    from oracle import stacks
    from sparse_attention_hub import workloads

    B, Hq, Hkv, D = 1, 32, 8, 128
    n = 8192
    stack = _long_stack(name, seed, Hq, D)
    q, k, v = workloads.qkv_clustered(seed, B, Hq, Hkv, n, D)
    q, k, v = (workloads.to_dtype(a, "bf16") for a in (q, k, v))
    meta: dict = {}
    if name == "magicpig":
        meta["lsh_projection"] = stack[-1][1]["projection"]
    t0 = time.perf_counter()
    stacks.run_stack(stack, q, k, v, 1.0 / np.sqrt(D), "bf16", meta=meta)  # builds the key-side state
    t_build = time.perf_counter() - t0
    keep = {kk: vv for kk, vv in meta.items() if kk in ("lsh_projection", "lsh_key_mean", "lsh_state", "hash_kcodes")}
    times = []
    t_start = time.perf_counter()
    while len(times) < 5 and (time.perf_counter() - t_start < budget_s or len(times) < 2):
        t0 = time.perf_counter()
        stacks.run_stack(stack, q, k, v, 1.0 / np.sqrt(D), "bf16", meta=dict(keep))
        times.append(time.perf_counter() - t0)
    per_step = float(np.median(times)) * (S / n)
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        cores = os.cpu_count() or 1
    return {"value": 1.0 / per_step, "unit": UNIT, "cores": int(cores), "kind": "port",
            "sample": (f"{name}: the first {n} of {S} keys (1 token/step), {len(times)} timed steady-state "
                       f"steps, median {np.median(times) * 1e3:.0f} ms, scaled by {S // n} (the restatement, "
                       f"like the reference, is dense in the key count); numpy on {cores} threads; "
                       f"key-side build {t_build:.1f} s not included"),
            "ms_per_step": per_step * 1e3, "steps": len(times)}


def run_long_native(args) -> None:
    import torch

    from sparse_attention_hub import _native, workloads
    from sparse_attention_hub.sparse_attention.research_attention.sharded import (
        DistComm, SequenceShardedAttention, plan_shards)
    from sparse_attention_hub.sparse_attention.utils import mask_attention_utils as mau

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the native path has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    _native.load()

    S_full, S_small = LONG_WORKLOADS[args.workload]
    S = S_small if args.small else S_full
    B, Hq, Hkv, D = 1, 32, 8, 128
    begin, end = plan_shards(S, world)[rank]
    stack = _long_stack(args.workload, args.seed, Hq, D)
    ra = workloads.research_attention(stack, "bf16", dev)
    k, v = workloads.clustered_kv_range(args.seed, B, Hkv, begin, end, D, dev, "bf16")
    q_np = workloads.to_dtype(workloads._rng(args.seed, 0).standard_normal((B, Hq, 1, D), dtype=np.float32), "bf16")
    q = workloads.to_torch(q_np, "bf16", dev)
    meta: dict = {}
    if args.workload == "magicpig":
        meta["projections"] = {0: workloads.to_torch(stack[-1][1]["projection"], "bf16", dev)}
    scaling = 1.0 / float(np.sqrt(D))
    if world > 1:
        sa = SequenceShardedAttention(ra, DistComm(), begin, S)

        def step(qq=q):
            return sa.custom_attention(None, qq, k, v, None, scaling, 0.0, sparse_meta_data=meta, layer_idx=0)[0]
    else:
        def step(qq=q):
            return ra.custom_attention(None, qq, k, v, None, scaling, 0.0, sparse_meta_data=meta, layer_idx=0)[0]

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    t0 = time.perf_counter()
    out = step()
    barrier()
    index_build_ms = (time.perf_counter() - t0) * 1e3
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def timed_loop(n_steps: int):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(n_steps)]
        for a, b in evs:
            flush.zero_()
            a.record()
            step()
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    for _ in range(max(args.warmup, 3)):
        step()
    launches0 = _native.launch_count()
    step()
    launches_per_step = _native.launch_count() - launches0
    barrier()
    eager_step = step
    launch_mode = "eager"
    graph = None
    if not args.eager:
        # One captured step (the collectives of a sharded step included); every rank captures
        # the same sequence of collectives, so the replays pair up like the eager calls do.
        from sparse_attention_hub.sparse_attention.research_attention.decode_graph import DecodeStepGraph

        graph = DecodeStepGraph(sa if world > 1 else ra, q, k, v, None, scaling, meta, layer_idx=0)
        launch_mode = "CUDA graph replay"

        def step(qq=None):
            return graph.replay(qq)

        barrier()
        for _ in range(3):
            step()
        barrier()
    with ClockSampler(local_rank, enabled=(rank == 0)) as clocks:
        barrier()   # rank 0 may have waited for the sampler's first line
        per_step_ms = timed_loop(args.steps)
    barrier()
    total_ms = float(sum(per_step_ms))

    # kernel-level times: a separate eager pass (timing events are not baked into the graph)
    graph_step = step
    step = eager_step
    barrier()
    eager_ms = float(sum(timed_loop(args.steps))) / args.steps
    _native.profile_enable(True)
    for slot in _native.PROFILE_SLOTS:
        _native.profile_read(slot)
    timed_loop(args.steps)
    prof = {slot: _native.profile_read(slot) for slot in _native.PROFILE_SLOTS}
    _native.profile_enable(False)
    step = graph_step
    barrier()

    ucount = mau.last_union_counts()
    union_rows = int(ucount.sum().item()) if ucount is not None else 0
    row_bytes = 2 * D * 2
    attn_bytes = union_rows * row_bytes + (q.numel() + out.numel()) * 2
    n_local = end - begin
    stage_bytes = {"attention": attn_bytes}
    if args.workload == "magicpig":
        stage_bytes["lsh_match"] = B * Hkv * n_local * 75
    else:
        stage_bytes["hash_topk"] = B * Hq * n_local * 4 * 2  # histogram pass + emit pass
    step_bytes = sum(stage_bytes.values())

    # end to end: query from pinned host memory, output back to the host
    q_host = torch.from_numpy(np.ascontiguousarray(q_np)).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(out.shape, dtype=torch.bfloat16).pin_memory()
    q_dev = torch.empty_like(q)

    if graph is not None:
        # the host copies are captured with the step: one replay reads the pinned query and
        # leaves the output in pinned host memory
        e2e_graph = DecodeStepGraph(sa if world > 1 else ra, q, k, v, None, scaling, meta, layer_idx=0,
                                    host_query=q_host, host_output=out_host)

        def e2e_step():
            e2e_graph.graph.replay()
            torch.cuda.synchronize()
    else:
        def e2e_step():
            q_dev.copy_(q_host, non_blocking=True)
            o = step(q_dev)
            out_host.copy_(o, non_blocking=True)
            torch.cuda.synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_times = []
    for _ in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        e2e_times.append(time.perf_counter() - t0)
    barrier()
    e2e_total = float(sum(e2e_times))

    stats = torch.tensor([total_ms, e2e_total, float(union_rows), float(step_bytes)], device=dev,
                         dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats, op=dist.ReduceOp.SUM)
        total_ms, e2e_total = float(mx[0].item()), float(mx[1].item())
    union_all, bytes_all = float(stats[2].item()), float(stats[3].item())

    if rank == 0:
        peaks = {}
        peaks_file = REPO / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peaks = json.loads(peaks_file.read_text())
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
        ms_per_step = total_ms / args.steps
        attn_ms, attn_n = prof["attention"]
        attn_avg_ms = attn_ms / max(attn_n, 1)
        achieved = attn_bytes / (attn_avg_ms * 1e-3) / 1e9 if attn_avg_ms > 0 else 0.0
        stage_times = {s: (ms / max(n, 1)) * 1e3 for s, (ms, n) in prof.items() if n > 0}
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base = long_cpu_baseline(args.workload, args.seed, S)
        cfg_stack = [{"masker": kind, **{a: b for a, b in prm.items() if a not in ("weights", "projection")}}
                     for kind, prm in stack]
        line = {
            "metric": METRIC, "value": B / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "us_per_layer": ms_per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": f"{args.workload}: B={B} Hq={Hq} Hkv={Hkv} Sq=1 S={S} D={D} bf16",
                "stack": cfg_stack, "seed_data": "synthetic, seeded (torch CUDA generator per 32768-key chunk)",
                "parallelism": (f"sequence-sharded over {world} GPU(s): {n_local} keys on rank 0; per step one "
                                "all-gather of (accumulator, max, denominator) per row" if world > 1
                                else "one GPU holds the whole sequence"),
                "l2": "flushed between steps (512 MiB memset outside the timed events)",
                "index_build_ms": index_build_ms, "launch": launch_mode,
                "eager_us_per_step_rank0": eager_ms * 1e3,
                "step_algorithmic_bytes_all_ranks": bytes_all,
                "step_hbm_fraction_of_measured_peak_per_gpu":
                    bytes_all / world / (ms_per_step * 1e-3) / 1e9 / hbm_peak,
                "union_rows_per_step_all_ranks": union_all,
                "selection_density": union_all / (B * Hkv * S),
                "kernel_us_rank0": stage_times,
            },
            "roofline": {
                "kernel": "masked_attention_kernel (K/V row gather + weighted online softmax), rank 0",
                "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak if hbm_peak else None, "peak_source": peak_src,
                "algorithmic_bytes_per_launch": attn_bytes, "avg_launch_us": attn_avg_ms * 1e3,
                "launches_timed": attn_n, "traffic": None,
            },
            "e2e": {"value": B / (e2e_total / args.steps), "unit": UNIT,
                    "h2d_bytes_per_step": int(q_host.numel() * 2), "d2h_bytes_per_step": int(out_host.numel() * 2),
                    "ms_per_step": e2e_total / args.steps * 1e3},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks.summary(),
        }
        if base is not None:
            line["cpu_baseline"] = {k_: base[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        import gc

        import torch.distributed as dist

        # graphs that captured collectives must be gone before their communicator is
        step = eager_step
        graph = e2e_graph = None  # noqa: F841
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


def run_long_reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    S_full, S_small = LONG_WORKLOADS[args.workload]
    S = S_small if args.small else S_full
    base = long_cpu_baseline(args.workload, args.seed, S, budget_s=60.0)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": base["steps"], "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: B=1 Hq=32 Hkv=8 Sq=1 S={S} D=128 bf16", "sample": base["sample"]},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="hashattention")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--small", action="store_true", help="reduced sizes (development only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="launch every step eagerly (no CUDA graph)")
    args = ap.parse_args()
    if args.workload in LONG_WORKLOADS:
        (run_long_reference_arm if args.impl == "reference" else run_long_native)(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
