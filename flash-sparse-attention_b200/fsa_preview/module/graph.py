"""A decode step replayed from a CUDA graph.

One step issues about a dozen short kernels; launched one by one from Python their host cost exceeds
their device time.  The step is free of host synchronisation and of data-dependent shapes (the cache is
pre-allocated, lengths live on the device, the compressor runs with masked writes), so it is captured
once and replayed: inputs are copied into fixed buffers, the output is read from a fixed buffer.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from fsa_preview.cache import DecodeCache


class GraphedStep:
    def __init__(self, fn: Callable[..., torch.Tensor], cache: DecodeCache, example_inputs: Sequence[torch.Tensor], warmup: int = 3):
        """``fn(*inputs, cache) -> tensor`` appends one token per sequence to ``cache``.  The warm-up runs before the
        capture advance the device-side lengths and overwrite ring slots of the compressor's input window; lengths
        and rings are put back afterwards, so the cache content is unchanged (rows past the length are scratch)."""
        self.cache = cache
        self.static_in = [t.clone() for t in example_inputs]
        cache.always_compress = True
        len0, host0 = cache.seq_len.clone(), list(cache.host_len)
        tails = cache.k_tail.clone(), cache.v_tail.clone()
        side = torch.cuda.Stream(device=cache.seq_len.device)
        side.wait_stream(torch.cuda.current_stream(cache.seq_len.device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                fn(*self.static_in, cache)
        torch.cuda.current_stream(cache.seq_len.device).wait_stream(side)
        cache.seq_len.copy_(len0)
        cache.k_tail.copy_(tails[0])
        cache.v_tail.copy_(tails[1])
        self.graph = torch.cuda.CUDAGraph()
        # thread_local: other threads of the process (a collective library's watchdog) may call into CUDA meanwhile
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"), torch.no_grad():
            self.static_out = fn(*self.static_in, cache)
        cache.seq_len.copy_(len0)                 # capture does not execute, but keep the invariant explicit
        cache.host_len = host0

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.cache.host_len = [L + 1 for L in self.cache.host_len]
        return self.static_out


class GraphedShardedAttention:
    """The KV-sequence-sharded decode attention as three CUDA graphs around its two all-gathers.

    A collective captured inside a graph did not complete, and launched kernel by kernel the sharded step is
    bound by host launch cost; so the step's three collective-free parts (``DecodeStepPlan.part1/2/3``) are captured
    separately and the two NCCL all-gathers of one packed buffer each stay ordinary launches between the replays:
    five launches per step instead of about forty."""

    def __init__(self, plan, q: torch.Tensor, cache: DecodeCache, finish: Callable[..., torch.Tensor], warmup: int = 2):
        import torch.distributed as dist

        self.dist, self.group = dist, plan.shard.group
        args1 = (q, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.cmp_row0)
        args2 = (q, cache.k, cache.v, cache.seq_len, cache.seq_row0)
        world = plan.shard.world
        with torch.no_grad():
            for _ in range(warmup):                          # eager: sizes the buffers, sets kernel attributes
                f1 = plan.part1(*args1)
                g1 = torch.empty(world * f1.numel(), dtype=f1.dtype, device=f1.device)
                dist.all_gather_into_tensor(g1, f1, group=self.group)
                f2 = plan.part2(*args2, g1)
                g2 = torch.empty(world * f2.numel(), dtype=f2.dtype, device=f2.device)
                dist.all_gather_into_tensor(g2, f2, group=self.group)
                finish(*plan.part3(q, g2)[:3])
            torch.cuda.synchronize()
            self.g1, self.g2 = g1, g2
            self.graph1, self.graph2, self.graph3 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph1, capture_error_mode="thread_local"):
                self.f1 = plan.part1(*args1)
            with torch.cuda.graph(self.graph2, capture_error_mode="thread_local"):
                self.f2 = plan.part2(*args2, self.g1)
            with torch.cuda.graph(self.graph3, capture_error_mode="thread_local"):
                self.out = finish(*plan.part3(q, self.g2)[:3])

    def __call__(self) -> torch.Tensor:
        self.graph1.replay()
        self.dist.all_gather_into_tensor(self.g1, self.f1, group=self.group)
        self.graph2.replay()
        self.dist.all_gather_into_tensor(self.g2, self.f2, group=self.group)
        self.graph3.replay()
        return self.out
