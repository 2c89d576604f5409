"""Decode-time sparse attention benchmark: one layer, one decode step per pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload: MagicPig LSH sampling at 1,048,576 keys in bf16 -- batch 1, 32 query / 8 KV
heads, head_dim 128, SimHash with 8 bits x 75 tables, Sink(64) + Local(256) -- with the KV
cache and the packed signatures sequence-sharded over the N GPUs (strong scaling: the same
sequence on every N).  A pass is the steady-state decode call of one layer through the public
API (`ResearchAttention.custom_attention`, or `SequenceShardedAttention.custom_attention`
over NCCL when N > 1): query hashing, signature match, union list, gather attention with the
sampling weights evaluated in the kernel, and for N > 1 one all-gather of the per-row
(accumulator, max, denominator) and their merge.  Signatures are built once before timing
(index build, reported separately).

Prints one JSON line (rank 0).  `value` is whole-job decode tokens per second per layer with
everything resident in HBM; `e2e` is the same through the public API with host buffers: the
query and one appended key/value row come from pinned host memory, the appended key is hashed
inside the step (with N > 1 that includes the ranks' agreement on the largest key norm), and
the output is read back to the host; it is timed with CUDA events around the copies and the step
(`e2e.wall_ms_per_step` is the host clock around replay + synchronise of the same step).  A
"step" of the command line is timed as `repeats`
passes back to back (L2 flushed before each), so that the timed region is at least 100 ms and
the clock sampler sees it; all times are per pass.

`--workload hashattention | sink_local | oracle_topk | oracle_adaptive | oracle_topp | quest |
pqcache` run the batch-sharded configurations (one batch per GPU, no collective, weak scaling);
`--workload hashattention_long` and `--workload pqcache_long` are the other sequence-sharded ones.

`--impl reference` times the reference's own `ResearchAttention.custom_attention` (CPU PyTorch,
from oracle/_ref, which oracle/make_ref.py makes) on the host cores on a bounded sample of the
same workload; where that package is absent, the numpy restatement in oracle/.
"""

from __future__ import annotations

import argparse
import json
import math
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
MIN_REGION_MS = 100.0

# name: (keys, keys with --small)
LONG_WORKLOADS = {"magicpig": (1048576, 65536), "hashattention_long": (1048576, 65536),
                  "pqcache_long": (262144, 65536)}
DEFAULT_WORKLOAD = "magicpig"
# keys of the long sequences that the reference is timed on (it is dense in the key count and
# materialises [B, Hq, S, L] int64 signatures: ~0.4 MB of temporaries per key)
REFERENCE_LONG_KEYS = 16384

# DRAM traffic per algorithmic byte of one launch (dram__bytes_read.sum + dram__bytes_write.sum
# over the bytes the kernel has to read), from ncu captures of the same kernel: the headline
# shape for HashAttention; for MagicPig the 65536-key case of the workload (the million-key
# launch is too large to capture under a profiler; traffic grows in proportion to the rows
# gathered).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {
    "hashattention": (221809920.0 + 4204032.0) / 219225088.0,        # masked_attention_mma_kernel
    "magicpig:attention": (200350976.0 + 4377856.0) / 196420096.0,   # masked_attention_umma_kernel
}


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
def make_workload(name: str, seed: int, small: bool = False):
    import workloads

    if name == "hashattention":
        if small:
            return workloads.hashattention_bf16(seed=seed, B=2, S=4096)
        if os.environ.get("SAH_BENCH_BATCH"):  # profiler captures use a smaller batch
            return workloads.hashattention_bf16(seed=seed, B=int(os.environ["SAH_BENCH_BATCH"]))
        return workloads.hashattention_bf16(seed=seed)
    if name == "sink_local":
        return workloads.sink_local_fp32(seed=seed)
    if name == "oracle_topk":
        return workloads.oracle_topk(seed=seed, B=1, S=8192) if small else workloads.oracle_topk(seed=seed)
    if name == "oracle_adaptive":
        return (workloads.oracle_adaptive(seed=seed, B=1, S=8192) if small
                else workloads.oracle_adaptive(seed=seed))
    if name == "oracle_topp":
        return workloads.oracle_topp(seed=seed, B=1, S=8192) if small else workloads.oracle_topp(seed=seed)
    if name == "quest":
        return workloads.quest(seed=seed, B=2, S=4096) if small else workloads.quest(seed=seed)
    if name == "pqcache":
        if small:
            return workloads.pqcache(seed=seed, S=16384, heavy=512, kmeans_iter=3)
        return workloads.pqcache(seed=seed)
    raise SystemExit(f"unknown workload {name}")


def long_stack(name: str, seed: int, Hq: int, D: int):
    import workloads

    if name == "magicpig":
        proj = workloads.to_dtype(
            workloads._rng(seed, 70).standard_normal((D + 1, 75 * 8)).astype(np.float32), "bf16")
        return [("sink", {"sink_size": 64}), ("local", {"window_size": 256}),
                ("magicpig", {"lsh_l": 75, "lsh_k": 8, "center": True, "projection": proj})]
    if name == "pqcache_long":
        return [("sink", {"sink_size": 64}), ("local", {"window_size": 256}),
                ("pq_topk", {"heavy_size": 2048, "pq_group_factor": 16, "pq_bits": 8, "kmeans_iter": 10,
                             "init_offset": 64, "metric": "euclidean"})]
    w = {n: [workloads.to_dtype(a, "bf16") for a in arrs]
         for n, arrs in workloads.hat_weights(seed, Hq, D, 128, 32, 3).items()}
    return [("sink", {"sink_size": 128}), ("local", {"window_size": 512}),
            ("hash_topk", {"heavy_size": 0.02, "bits": 32, "hidden": 128, "layers": 3,
                           "activation": "silu", "weights": w})]


def stack_config(stack) -> list:
    return [{"masker": kind, **{a: b for a, b in prm.items() if a not in ("weights", "projection")}}
            for kind, prm in stack]


def workload_config(wl, name: str, extra: dict) -> dict:
    B, Hq, Hkv, Sq, S, D = wl.shape
    cfg = {"workload": f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq={Sq} S={S} D={D} {wl.dtype}",
           "stack": stack_config(wl.stack), "seed_data": "synthetic, seeded (numpy Philox)"}
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
                 "-lms", "20", "-i", str(self.index)],
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
# the reference arm and the CPU baseline
# ---------------------------------------------------------------------------
def _host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def reference_baseline(name: str, seed: int, small: bool, steps: int, warmup: int,
                       budget_s: float) -> dict:
    """The reference's own `custom_attention` (CPU PyTorch) from oracle/_ref, steady-state
    decode after the index build: whole batch for the batch-sharded workloads, the first
    REFERENCE_LONG_KEYS keys for the long ones (time scaled by the key ratio)."""
    ref_dir = REPO / "oracle" / "_ref"
    sys.path.insert(0, str(ref_dir))
    import torch

    import workloads
    import sparse_attention_hub as ref_pkg

    if Path(ref_pkg.__file__).resolve().parent.parent != ref_dir.resolve():
        raise RuntimeError("the reference arm must import the reference package, found "
                           f"{ref_pkg.__file__}")
    threads = _host_threads()
    torch.set_num_threads(threads)
    meta: dict = {}
    if name in LONG_WORKLOADS:
        S_full = LONG_WORKLOADS[name][1 if small else 0]
        S = min(S_full, 8192 if small else int(os.environ.get("SAH_REF_KEYS", REFERENCE_LONG_KEYS)))
        B, Hq, Hkv, D = 1, 32, 8, 128
        stack = long_stack(name, seed, Hq, D)
        k, v = workloads.clustered_kv_range(seed, B, Hkv, 0, S, D, "cpu", "bf16")
        q = workloads.to_torch(workloads.to_dtype(
            workloads._rng(seed, 0).standard_normal((B, Hq, 1, D), dtype=np.float32), "bf16"), "bf16", "cpu")
        dtype, scaling, tokens, scale = "bf16", 1.0 / math.sqrt(D), B, S_full / S
        if name == "magicpig":
            meta["projections"] = {0: workloads.to_torch(stack[-1][1]["projection"], "bf16", "cpu")}
        shape_txt = f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq=1 S={S_full} D={D} bf16"
        sample_txt = (f"the first {S} of {S_full} keys (the reference is dense in the key count and "
                      f"cannot hold its int64 signature tensors for more); time scaled by {scale:g}")
    else:
        wl = make_workload(name, seed, small)
        B, Hq, Hkv, Sq, S, D = wl.shape
        stack, dtype, scaling, tokens, scale = wl.stack, wl.dtype, float(wl.scaling), B, 1.0
        q, k, v = (workloads.to_torch(a, dtype, "cpu") for a in (wl.q, wl.k, wl.v))
        shape_txt = f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq={Sq} S={S} D={D} {dtype}"
        sample_txt = f"the whole batch of {B}"
    ra = workloads.research_attention(stack, dtype, "cpu")

    def step():
        with torch.no_grad():
            return ra.custom_attention(None, q, k, v, None, scaling, 0.0, sparse_meta_data=meta,
                                       layer_idx=0)[0]

    t0 = time.perf_counter()
    step()  # builds the key-side state (signatures, hash codes)
    t_build = time.perf_counter() - t0
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
    per_step = float(np.median(times)) * scale
    return {"value": tokens / per_step, "unit": UNIT, "cores": threads, "kind": "reference",
            "sample": (f"{sample_txt}; {len(times)} timed steady-state calls of the reference's "
                       f"ResearchAttention.custom_attention (CPU PyTorch {torch.__version__}, "
                       f"{threads} threads), median {np.median(times) * 1e3:.1f} ms; first call "
                       f"(index build) {t_build:.1f} s not included"),
            "ms_per_step": per_step * 1e3, "steps": len(times), "workload": shape_txt,
            "stack": stack_config(stack), "dtype": dtype}


def port_baseline(name: str, seed: int, small: bool, steps: int, warmup: int, budget_s: float) -> dict:
    """The numpy restatement (oracle/) where the reference package is absent or cannot run
    the workload in bounded time (PQCache: its k-means build): batch element 0, or the first
    8192 keys of a long sequence."""
    from oracle import attention as o_attn, hashattention as o_hash, stacks
    import workloads

    try:
        from threadpoolctl import threadpool_info
        threads = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        threads = _host_threads()
    meta: dict = {}
    if name in LONG_WORKLOADS:
        S_full = LONG_WORKLOADS[name][1 if small else 0]
        S = min(S_full, 8192)
        B, Hq, Hkv, D = 1, 32, 8, 128
        stack = long_stack(name, seed, Hq, D)
        q, k, v = (workloads.to_dtype(a, "bf16") for a in workloads.qkv_clustered(seed, B, Hq, Hkv, S, D))
        dtype, scaling, scale = "bf16", 1.0 / np.sqrt(D), S_full / S
        if name == "magicpig":
            meta["lsh_projection"] = stack[-1][1]["projection"]
        shape_txt = f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq=1 S={S_full} D={D} bf16"
        sample_txt = f"the first {S} of {S_full} keys, time scaled by {scale:g}"
    else:
        wl = make_workload(name, seed, small)
        B, Hq, Hkv, Sq, S, D = wl.shape
        q, k, v = wl.q[:1], wl.k[:1], wl.v[:1]
        stack, dtype, scaling, scale = wl.stack, wl.dtype, wl.scaling, 1.0
        shape_txt = f"{name}: B={B} Hq={Hq} Hkv={Hkv} Sq={Sq} S={S} D={D} {dtype}"
        sample_txt = "batch element 0 (1 token per call)"
    for kind, prm in stack:
        if kind == "hash_topk":
            G = q.shape[1] // k.shape[1]
            w = prm["weights"]
            meta["hash_kcodes"] = o_hash.signatures_blas(o_attn.repeat_kv(k, G), w["key_matrix"],
                                                         w["key_bias"], prm["activation"], dtype)
        if kind == "pq_topk":
            # The decode step's cost does not depend on how good the codebook is: centres are
            # the seeded initial keys (no Lloyd iteration), codes their nearest-centre assignment.
            from oracle import pq as o_pq
            from oracle.bf16 import round_to
            off, n_sub, cent = prm["init_offset"], prm["pq_group_factor"], 2 ** prm["pq_bits"]
            X = o_pq.split_keys(k, off, n_sub)
            idx = workloads.pq_init_indices(0, X.shape[0], X.shape[1], cent)
            C = X[np.arange(X.shape[0])[:, None], idx]
            codes = np.concatenate([o_pq.assign(X[g:g + 1], C[g:g + 1]) for g in range(X.shape[0])])
            Hkv_, n_ = k.shape[1], X.shape[1]
            meta["pq_centroids"] = round_to(C, dtype).reshape(1, Hkv_, n_sub, cent, -1)
            meta["pq_codes"] = codes.reshape(1, Hkv_, n_sub, n_).transpose(0, 1, 3, 2)
        if kind == "adaptive_sampling":
            meta["adaptive_seed"] = 0
    t0 = time.perf_counter()
    if name in LONG_WORKLOADS:
        stacks.run_stack(stack, q, k, v, scaling, dtype, meta=meta)  # builds the key-side state
        meta = {kk: vv for kk, vv in meta.items()
                if kk in ("lsh_projection", "lsh_key_mean", "lsh_state", "hash_kcodes")}
    t_build = time.perf_counter() - t0
    times = []
    t_start = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        stacks.run_stack(stack, q, k, v, scaling, dtype, meta=dict(meta))
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_start > budget_s and len(times) >= 2:
            break
    per_step = float(np.median(times)) * scale
    return {"value": 1.0 / per_step, "unit": UNIT, "cores": int(threads), "kind": "port",
            "sample": (f"{sample_txt}; {len(times)} timed steady-state steps of the numpy restatement "
                       f"of the reference algorithm (dense in the key count), BLAS on {threads} "
                       f"threads, median {np.median(times) * 1e3:.1f} ms; key-side build "
                       f"{t_build:.1f} s not included"),
            "ms_per_step": per_step * 1e3, "steps": len(times), "workload": shape_txt,
            "stack": stack_config(stack), "dtype": dtype}


# workloads whose reference run cannot be bounded (PQCache's CPU k-means takes hours at this size)
PORT_ONLY = {"pqcache"}


def cpu_arm(name: str, seed: int, small: bool, steps: int, warmup: int, budget_s: float) -> dict:
    have_ref = (REPO / "oracle" / "_ref" / "sparse_attention_hub" / "__init__.py").exists()
    if have_ref and name not in PORT_ONLY:
        try:
            return reference_baseline(name, seed, small, steps, warmup, budget_s)
        except Exception as exc:  # e.g. a masker the reference package does not have
            sys.stderr.write(f"reference package could not run {name} ({exc!r}); using the restatement\n")
    return port_baseline(name, seed, small, steps, warmup, budget_s)


def run_reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    base = cpu_arm(args.workload, args.seed, args.small, args.steps, args.warmup, args.budget)
    long = args.workload in LONG_WORKLOADS
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT,
        "n_gpus": args.gpus, "steps": base["steps"], "warmup": args.warmup,
        "ms_per_step": base["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if long else "weak", "vs_baseline": None, "dtype": base["dtype"],
        "data": "synthetic",
        "config": {"workload": base["workload"], "stack": base["stack"], "sample": base["sample"]},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)


def cpu_baseline_subprocess(args, budget_s: float = 25.0):
    """The reference arm as a child process (the reference package has the same import name as
    the one under test, so the two cannot share an interpreter)."""
    cmd = [sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--workload", args.workload,
           "--seed", str(args.seed), "--steps", "8", "--warmup", "1", "--budget", str(budget_s)]
    if args.small:
        cmd.append("--small")
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT")}
    env["CUDA_VISIBLE_DEVICES"] = ""
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for line in reversed(res.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)["cpu_baseline"]
        sys.stderr.write("cpu baseline: no result line\n" + res.stderr[-2000:])
    except (subprocess.TimeoutExpired, OSError, ValueError) as exc:
        sys.stderr.write(f"cpu baseline failed: {exc!r}\n")
    return None


# ---------------------------------------------------------------------------
# timing helpers of the native arms
# ---------------------------------------------------------------------------
def _peaks():
    peaks = {}
    peaks_file = REPO / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peaks = json.loads(peaks_file.read_text())
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
    return hbm, src


class PassTimer:
    """CUDA-event timing of decode passes on the current stream, L2 flushed before each."""

    def __init__(self, torch, dev):
        self.torch = torch
        self.flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > L2 (126 MB)

    def run(self, fn, n: int):
        torch = self.torch
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(n)]
        for a, b in evs:
            self.flush.zero_()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]


def _repeats(est_ms: float, steps: int) -> int:
    return max(1, int(math.ceil(MIN_REGION_MS / max(est_ms * steps, 1e-6))))


# ---------------------------------------------------------------------------
# batch-sharded workloads (one batch per GPU, no collective)
# ---------------------------------------------------------------------------
def run_native(args) -> None:
    import torch

    import workloads
    from sparse_attention_hub import _native
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

    def eager_step(qq=q):
        return ra.custom_attention(None, qq, k, v, None, scaling, 0.0, sparse_meta_data=meta,
                                   layer_idx=0)[0]

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # index build (first call hashes every key); timed on its own
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = eager_step()
    torch.cuda.synchronize()
    index_build_ms = (time.perf_counter() - t0) * 1e3
    timer = PassTimer(torch, dev)

    # The decode step is captured once and replayed as a CUDA graph (public API:
    # sparse_attention_hub...research_attention.decode_graph.DecodeStepGraph).
    from sparse_attention_hub.sparse_attention.research_attention.decode_graph import DecodeStepGraph
    step = eager_step
    if not args.eager:
        graph = DecodeStepGraph(ra, q, k, v, None, scaling, meta, layer_idx=0)

        def step():  # noqa: F811
            return graph.replay(None)

    warm = timer.run(step, max(args.warmup, 3))
    launches0 = _native.launch_count()
    eager_step()
    launches_per_pass = _native.launch_count() - launches0
    torch.cuda.synchronize()
    est = torch.tensor([float(np.median(warm))], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    repeats = _repeats(float(est.item()), args.steps)
    passes = args.steps * repeats
    barrier()
    with ClockSampler(local_rank, enabled=(rank == 0)) as clocks:
        barrier()   # rank 0 may have waited for the sampler's first line
        per_pass_ms = timer.run(step, passes)
    barrier()
    total_ms = float(sum(per_pass_ms))

    # kernel-level times: a separate eager pass, so that the timing events neither sit
    # inside `value` nor get baked into the graph
    eager_ms = float(np.mean(timer.run(eager_step, args.steps)))
    _native.profile_enable(True)
    for slot in _native.PROFILE_SLOTS:
        _native.profile_read(slot)

    def probed():
        eager_step()
        if wl.dtype == "bf16":
            mau.gather_probe(k, v, Sq)

    timer.run(probed, args.steps)
    prof = {slot: _native.profile_read(slot) for slot in _native.PROFILE_SLOTS}
    _native.profile_enable(False)

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
        # same public call, captured with "one key appended since the last call"; the three
        # host-to-device copies and the read-back are nodes of the same graph
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

    for _ in range(3):
        e2e_step()
        torch.cuda.synchronize()
    barrier()
    # Device time of the end-to-end step: events on the launching stream around the replay
    # (H2D copies, the step, the D2H copy), the L2 flush directly in front of the first event.
    # The wall clock of the same steps (launch latency and the wake-up of the synchronising
    # host thread included) is reported beside it.
    e2e_times, e2e_events = [], []
    for _ in range(passes):
        timer.flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        torch.cuda.synchronize()
        e2e_times.append(time.perf_counter() - t0)
    barrier()
    for _ in range(passes):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        timer.flush.zero_()
        ev0.record()
        e2e_step()
        ev1.record()
        e2e_events.append((ev0, ev1))
    barrier()
    e2e_wall_total = float(sum(e2e_times))
    e2e_total = float(sum(a.elapsed_time(b) for a, b in e2e_events)) * 1e-3

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([total_ms, e2e_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_total = float(t[0].item()), float(t[1].item())

    if rank == 0:
        hbm_peak, peak_src = _peaks()
        from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import last_attention_kernel
        attention_kernel_name = last_attention_kernel()
        ms_per_pass = total_ms / passes
        tokens = B * world
        attn_ms, attn_n = prof["attention"]
        attn_avg_ms = attn_ms / max(attn_n, 1)
        achieved = attn_bytes / (attn_avg_ms * 1e-3) / 1e9 if attn_avg_ms > 0 else 0.0
        probe_ms, probe_n = prof["other"]
        probe_gbs = (union_rows * row_bytes / (probe_ms / probe_n * 1e-3) / 1e9) if probe_n else None
        stage_times = {s: (ms / max(n, 1)) * 1e3 for s, (ms, n) in prof.items() if n > 0 and s != "other"}
        ratio = None if args.small else NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(args.workload)
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_baseline_subprocess(args)
        line = {
            "metric": METRIC,
            "value": tokens / (ms_per_pass * 1e-3),
            "unit": UNIT,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_pass,
            "us_per_layer": ms_per_pass * 1e3,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": wl.dtype,
            "data": "synthetic",
            "config": workload_config(wl, args.workload, {
                "parallelism": f"dp{world} (one batch per GPU, no data-path collective)",
                "l2": "flushed before every pass (512 MiB memset outside the timed events)",
                "repeats": repeats, "timed_passes": passes, "timed_region_ms": total_ms,
                "index_build_ms": index_build_ms,
                "launch": "eager" if args.eager else "CUDA graph replay of the public decode call",
                "eager_ms_per_step": eager_ms,
                "step_algorithmic_bytes": step_bytes,
                "step_hbm_fraction_of_measured_peak":
                    step_bytes / (ms_per_pass * 1e-3) / 1e9 / hbm_peak,
                "union_rows_per_step": union_rows,
                "kernel_us": stage_times,
            }),
            "roofline": {
                "kernel": f"{attention_kernel_name} (K/V row gather + weighted online softmax)",
                "bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak if hbm_peak else None, "peak_source": peak_src,
                "frac_of_nominal_8TBs": achieved / 8000.0,
                "algorithmic_bytes_per_launch": attn_bytes,
                "avg_launch_us": attn_avg_ms * 1e3, "launches_timed": attn_n,
                "traffic": attn_bytes * ratio if ratio else None,
                "traffic_source": ("ncu capture of one launch of the mma.sync attention kernel on this "
                                   "workload's union list (read + write), scaled by the algorithmic "
                                   "bytes of the timed launch") if ratio else None,
                "gather_only_gbs": probe_gbs,
            },
            "e2e": {
                "value": tokens / (e2e_total / passes), "unit": UNIT,
                "h2d_bytes_per_step": int((q_host.numel() + kn_host.numel() + vn_host.numel()) * esz),
                "d2h_bytes_per_step": int(out_host.numel() * esz),
                "ms_per_step": e2e_total / passes * 1e3,
                "wall_ms_per_step": e2e_wall_total / passes * 1e3,
                "timing": "CUDA events around H2D copies + step + D2H copy; wall_ms_per_step is the host clock "
                          "around replay + synchronise of the same step",
            },
            "gpu_launches": int(launches_per_pass * passes),
            "clocks": clocks.summary(),
        }
        if base is not None:
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# long-context workloads: the KV cache is sequence-sharded over the GPUs (strong scaling)
# ---------------------------------------------------------------------------
def run_long_native(args) -> None:
    import torch

    import workloads
    from sparse_attention_hub import _native
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
    if args.keys:
        S = int(args.keys)
    B, Hq, Hkv, D = 1, 32, 8, 128
    begin, end = plan_shards(S, world)[rank]
    n_local = end - begin
    stack = long_stack(args.workload, args.seed, Hq, D)
    ra = workloads.research_attention(stack, "bf16", dev)
    k, v = workloads.clustered_kv_range(args.seed, B, Hkv, begin, end, D, dev, "bf16")
    q_np = workloads.to_dtype(workloads._rng(args.seed, 0).standard_normal((B, Hq, 1, D), dtype=np.float32), "bf16")
    q = workloads.to_torch(q_np, "bf16", dev)
    meta: dict = {}
    if args.workload == "magicpig":
        meta["projections"] = {0: workloads.to_torch(stack[-1][1]["projection"], "bf16", dev)}
    scaling = 1.0 / float(np.sqrt(D))

    class TimedComm(DistComm):
        """DistComm that brackets every collective with CUDA events while `timing` is on."""

        def __init__(self):
            super().__init__()
            self.timing = False
            self.records = []

        def _timed(self, name, fn, t):
            if not self.timing:
                return fn(t)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            r = fn(t)
            b.record()
            self.records.append((name, a, b))
            return r

        def all_reduce_sum_(self, t):
            return self._timed("all_reduce_sum", super().all_reduce_sum_, t)

        def all_reduce_max_(self, t):
            return self._timed("all_reduce_max", super().all_reduce_max_, t)

        def all_gather(self, t):
            return self._timed(f"all_gather_{t.numel() * t.element_size()}B", super().all_gather, t)

        def per_step_us(self, n_steps: int) -> dict:
            torch.cuda.synchronize()
            out: dict = {}
            for name, a, b in self.records:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b) * 1e3 / n_steps
            self.records = []
            return out

    comm = TimedComm() if world > 1 else None
    attn = SequenceShardedAttention(ra, comm, begin, S) if world > 1 else ra

    def eager_step(qq=q):
        return attn.custom_attention(None, qq, k, v, None, scaling, 0.0, sparse_meta_data=meta,
                                     layer_idx=0)[0]

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    t0 = time.perf_counter()
    out = eager_step()
    barrier()
    index_build_ms = (time.perf_counter() - t0) * 1e3
    timer = PassTimer(torch, dev)

    for _ in range(3):
        eager_step()
    launches0 = _native.launch_count()
    eager_step()
    launches_per_pass = _native.launch_count() - launches0
    barrier()
    step = eager_step
    launch_mode = "eager"
    graph = e2e_graph = None
    from sparse_attention_hub.sparse_attention.research_attention.decode_graph import DecodeStepGraph
    if not args.eager:
        # One captured step (the collectives of a sharded step included); every rank captures
        # the same sequence of collectives, so the replays pair up like the eager calls do.
        graph = DecodeStepGraph(attn, q, k, v, None, scaling, meta, layer_idx=0)
        launch_mode = "CUDA graph replay"

        def step():  # noqa: F811
            return graph.replay(None)

        barrier()
    warm = timer.run(step, max(args.warmup, 3))
    est = torch.tensor([float(np.median(warm))], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    repeats = _repeats(float(est.item()), args.steps)
    passes = args.steps * repeats
    barrier()
    with ClockSampler(local_rank, enabled=(rank == 0)) as clocks:
        barrier()   # rank 0 may have waited for the sampler's first line
        per_pass_ms = timer.run(step, passes)
    barrier()
    total_ms = float(sum(per_pass_ms))

    # kernel-level and per-collective times: a separate eager pass (timing events are not baked
    # into the graph)
    barrier()
    eager_ms = float(np.mean(timer.run(eager_step, args.steps)))
    _native.profile_enable(True)
    for slot in _native.PROFILE_SLOTS:
        _native.profile_read(slot)
    if comm is not None:
        comm.timing = True

    def probed():
        eager_step()
        mau.gather_probe(k, v, 1)

    timer.run(probed, args.steps)
    prof = {slot: _native.profile_read(slot) for slot in _native.PROFILE_SLOTS}
    collective_us = comm.per_step_us(args.steps) if comm is not None else {}
    if comm is not None:
        comm.timing = False
    _native.profile_enable(False)
    barrier()

    ucount = mau.last_union_counts()
    union_rows = int(ucount.sum().item()) if ucount is not None else 0
    row_bytes = 2 * D * 2
    attn_bytes = union_rows * row_bytes + (q.numel() + out.numel()) * 2
    stage_bytes = {"attention": attn_bytes}
    if args.workload == "magicpig":
        stage_bytes["lsh_match"] = B * Hkv * n_local * 75
    elif args.workload == "pqcache_long":
        stage_bytes["pq_scores"] = B * Hkv * n_local * 16  # one code byte per sub-vector
    else:
        stage_bytes["hash_topk"] = B * Hq * n_local * 4  # the packed codes, once
    step_bytes = sum(stage_bytes.values())

    # End to end: the query and one appended key/value row (on the rank that owns the end of
    # the sequence) come from pinned host memory; the appended key is hashed inside the step,
    # which for a sharded MagicPig index includes the ranks' agreement on the largest key
    # norm; the output goes back to pinned host memory.
    last = rank == world - 1
    q_host = torch.from_numpy(np.ascontiguousarray(q_np)).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(out.shape, dtype=torch.bfloat16).pin_memory()
    kn_host = k[:, :, n_local - 1:, :].cpu().pin_memory()
    vn_host = v[:, :, n_local - 1:, :].cpu().pin_memory()
    host_inputs = [(k[:, :, n_local - 1:, :], kn_host), (v[:, :, n_local - 1:, :], vn_host)] if last else []
    sig = meta.get("key_signature", {}).get(0)
    key_cache = meta.get("key", {}).get(0)
    pq_codes = meta.get("pq_codebook", {}).get(0)

    def mark_appended():
        if sig is not None:       # MagicPig: PackedLSHSignatures
            if last:
                sig.length = n_local - 1
            sig.synced_total = None  # keys arrived somewhere: the maximum norm is agreed on again
        if key_cache is not None and last:  # HashAttention: packed key codes
            key_cache.length = n_local - 1
        if pq_codes is not None and last:   # PQCache: the appended key is quantised inside the step
            pq_codes.length -= 1

    q_dev = torch.empty_like(q)
    if not args.eager:
        e2e_graph = DecodeStepGraph(attn, q, k, v, None, scaling, meta, layer_idx=0,
                                    before_each_call=mark_appended, host_query=q_host,
                                    host_inputs=host_inputs,
                                    host_output=out_host if rank == 0 else None)

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.graph.replay()
        else:
            for dst, src in host_inputs:
                dst.copy_(src, non_blocking=True)
            q_dev.copy_(q_host, non_blocking=True)
            mark_appended()
            o = eager_step(q_dev)
            if rank == 0:
                out_host.copy_(o, non_blocking=True)

    for _ in range(3):
        e2e_step()
        torch.cuda.synchronize()
    barrier()
    # Device time of the end-to-end step: events on the launching stream around the replay
    # (H2D copies, the step, the D2H copy), the L2 flush directly in front of the first event.
    # The wall clock of the same steps (launch latency and the wake-up of the synchronising
    # host thread included) is reported beside it.
    e2e_times, e2e_events = [], []
    for _ in range(passes):
        timer.flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_step()
        torch.cuda.synchronize()
        e2e_times.append(time.perf_counter() - t0)
    barrier()
    for _ in range(passes):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        timer.flush.zero_()
        ev0.record()
        e2e_step()
        ev1.record()
        e2e_events.append((ev0, ev1))
    barrier()
    e2e_wall_total = float(sum(e2e_times))
    e2e_total = float(sum(a.elapsed_time(b) for a, b in e2e_events)) * 1e-3

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
        hbm_peak, peak_src = _peaks()
        ms_per_pass = total_ms / passes
        stage_times = {s: (ms / max(n, 1)) * 1e3 for s, (ms, n) in prof.items() if n > 0 and s != "other"}
        probe_ms, probe_n = prof["other"]
        probe_gbs = (union_rows * row_bytes / (probe_ms / probe_n * 1e-3) / 1e9) if probe_n else None
        # the roofline object describes the kernel that takes the largest share of the pass
        from sparse_attention_hub.sparse_attention.utils.mask_attention_utils import last_attention_kernel
        names = {"attention": f"{last_attention_kernel()} (K/V row gather + weighted online softmax, "
                              "MagicPig weights evaluated in place)" if args.workload == "magicpig"
                              else f"{last_attention_kernel()} (K/V row gather + online softmax)",
                 "lsh_match": "lsh_match_kernel (stream of the packed SimHash signatures)",
                 "hash_topk": "hash_hist + hash_emit (stream of the packed hash codes)",
                 "pq_scores": "pq_scores_kernel (stream of the product-quantisation codes)"}
        dom = max((s for s in stage_bytes if s in stage_times), key=lambda s: stage_times[s])
        dom_us = stage_times[dom]
        achieved = stage_bytes[dom] / (dom_us * 1e-6) / 1e9 if dom_us > 0 else 0.0
        base = None
        if world == 1 and not args.no_cpu_baseline:
            base = cpu_baseline_subprocess(args)
        ratio = None if (args.small or args.keys) else NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(f"{args.workload}:{dom}")
        line = {
            "metric": METRIC, "value": B / (ms_per_pass * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_pass,
            "us_per_layer": ms_per_pass * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": f"{args.workload}: B={B} Hq={Hq} Hkv={Hkv} Sq=1 S={S} D={D} bf16",
                "stack": stack_config(stack),
                "seed_data": "synthetic, seeded (torch CUDA generator per 32768-key chunk)",
                "parallelism": (f"sequence-sharded over {world} GPUs ({n_local} keys on rank 0); per pass one "
                                "NCCL all-gather of (accumulator, max, denominator) per row" if world > 1
                                else "one GPU holds the whole sequence"),
                "l2": "flushed before every pass (512 MiB memset outside the timed events)",
                "repeats": repeats, "timed_passes": passes, "timed_region_ms": total_ms,
                "index_build_ms": index_build_ms, "launch": launch_mode,
                "eager_us_per_step_rank0": eager_ms * 1e3,
                "step_algorithmic_bytes_all_ranks": bytes_all,
                "step_hbm_fraction_of_measured_peak_per_gpu":
                    bytes_all / world / (ms_per_pass * 1e-3) / 1e9 / hbm_peak,
                "union_rows_per_step_all_ranks": union_all,
                "selection_density": union_all / (B * Hkv * S),
                "kernel_us_rank0": stage_times,
                "collective_us": collective_us,
            },
            "roofline": {
                "kernel": names[dom] + ", rank 0", "bound": "hbm", "achieved": achieved,
                "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak if hbm_peak else None,
                "peak_source": peak_src, "frac_of_nominal_8TBs": achieved / 8000.0,
                "algorithmic_bytes_per_launch": stage_bytes[dom], "avg_launch_us": dom_us,
                "launches_timed": prof[dom][1],
                "traffic": stage_bytes[dom] * ratio if ratio else None,
                "traffic_source": ("ncu capture of a 65536-key launch of this kernel (read + write), "
                                   "scaled by the algorithmic bytes of the timed launch") if ratio else None,
                "gather_only_gbs": probe_gbs,
            },
            "e2e": {"value": B / (e2e_total / passes), "unit": UNIT,
                    "h2d_bytes_per_step": int(q_host.numel() * 2 * world + (kn_host.numel() + vn_host.numel()) * 2),
                    "d2h_bytes_per_step": int(out_host.numel() * 2),
                    "ms_per_step": e2e_total / passes * 1e3,
                    "wall_ms_per_step": e2e_wall_total / passes * 1e3,
                    "timing": "CUDA events around H2D copies + step + D2H copy (maximum over ranks); "
                              "wall_ms_per_step is rank 0's host clock around replay + synchronise"},
            "gpu_launches": int(launches_per_pass * passes),
            "clocks": clocks.summary(),
        }
        if base is not None:
            line["cpu_baseline"] = base
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--small", action="store_true", help="reduced sizes (development only)")
    ap.add_argument("--keys", type=int, default=0,
                    help="sequence length of the sequence-sharded workloads (development only)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="launch every step eagerly (no CUDA graph)")
    ap.add_argument("--budget", type=float, default=150.0,
                    help="seconds of timed CPU work of the reference arm")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload in LONG_WORKLOADS:
        run_long_native(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
