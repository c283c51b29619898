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
