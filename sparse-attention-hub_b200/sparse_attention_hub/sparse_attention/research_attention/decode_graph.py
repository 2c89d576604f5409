"""CUDA-graph replay of one decode step.

A decode step of a masker stack is a handful of short kernels (hash the query,
select, plan, gather attention); at 32K keys the whole step is tens of
microseconds, the same order as the host cost of launching it.  Capturing the
step once and replaying the graph removes that host cost.  The step's tensors
must keep their addresses between replays: the KV cache is used in place, the
query lives in a buffer owned by the graph object.

    graph = DecodeStepGraph(attention, queries, keys, values, None, scaling,
                            sparse_meta_data, layer_idx=0)
    out = graph.replay(new_queries)        # [B, Sq, Hq, D], valid on the current stream

The capture runs the public `ResearchAttention.custom_attention` unchanged, so
whatever that call would do for the captured key length (including hashing keys
appended since the previous call) is what each replay does.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch


class DecodeStepGraph:
    """One captured `custom_attention` call with pointer-stable inputs."""

    def __init__(self, attention, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                 attention_mask: Optional[torch.Tensor], scaling: float,
                 sparse_meta_data: Dict[Any, Any], layer_idx: int = 0, warmup: int = 2,
                 before_each_call: Optional[Callable[[], None]] = None,
                 host_query: Optional[torch.Tensor] = None, host_inputs=(),
                 host_output: Optional[torch.Tensor] = None, **kwargs: Any) -> None:
        if not queries.is_cuda:
            raise RuntimeError("DecodeStepGraph needs CUDA tensors")
        self.attention = attention
        self.queries = queries.clone()
        self.keys, self.values = keys, values
        self.attention_mask = attention_mask
        self.scaling = float(scaling)
        self.meta = sparse_meta_data
        self.kwargs = dict(kwargs, layer_idx=layer_idx)
        self._before = before_each_call
        # Optional host side of the step, captured with it: the query is read from a pinned
        # host tensor, `host_inputs` = [(device view, pinned host tensor), ...] are copied in
        # first (e.g. the appended K/V rows), and the output is copied to a pinned host tensor.
        # The caller rewrites the pinned tensors in place between replays.
        self.host_query, self.host_inputs, self.host_output = host_query, list(host_inputs), host_output
        for t in [host_query, host_output] + [h for _, h in self.host_inputs]:
            if t is not None and not t.is_pinned():
                raise RuntimeError("host tensors of a captured step must be pinned")

        def call() -> torch.Tensor:
            if self._before is not None:
                self._before()
            if self.host_query is not None:
                self.queries.copy_(self.host_query, non_blocking=True)
            for dst, src in self.host_inputs:
                dst.copy_(src, non_blocking=True)
            out, _ = self.attention.custom_attention(
                None, self.queries, self.keys, self.values, self.attention_mask, self.scaling, 0.0,
                sparse_meta_data=self.meta, **self.kwargs)
            if self.host_output is not None:
                self.host_output.copy_(out, non_blocking=True)
            return out

        # Warm up on a side stream: fills the workspaces, tables and signature caches
        # that must already exist when the capture starts.
        side = torch.cuda.Stream(device=queries.device)
        side.wait_stream(torch.cuda.current_stream(queries.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                call()
        torch.cuda.current_stream(queries.device).wait_stream(side)
        torch.cuda.synchronize(queries.device)

        # The attention scratch is cached per (stream, shape): capture on the warm-up stream so
        # that the capture finds it, and keep it alive for as long as the graph may replay.
        from ..utils import mask_attention_utils

        self._scratch = list(mask_attention_utils._workspace_cache.values())
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            self.out = call()

    def replay(self, queries: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy `queries` into the captured buffer (if given) and replay; returns the output buffer."""
        if queries is not None:
            self.queries.copy_(queries, non_blocking=True)
        self.graph.replay()
        return self.out
