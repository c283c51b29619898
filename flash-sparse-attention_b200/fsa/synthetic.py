"""Seeded synthetic workloads for the selected-attention path (benchmarks and tests).

The reference's own benchmark inputs are ``torch.randn`` with seed 42
(test/test_FSA_optimized_sel_attn.py:61-71); block indices there come from the compressed
branch.  For the bare operator the generator below produces indices with the same contract
(``topk_idx[Hk, N, T]`` int32, per-sequence-local block ids, ascending, -1 padded at the tail,
nsa_ref/ops/compressed_attention.py:1309-1313): for token ``t`` in block ``b = t_local //
block_size`` the set is ``{0, b}`` plus a uniform sample without replacement from ``1..b-1``.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np
import torch


def make_cu_seqlens(seqlens: Sequence[int]) -> torch.Tensor:
    cu = np.zeros(len(seqlens) + 1, dtype=np.int32)
    cu[1:] = np.cumsum(np.asarray(seqlens, dtype=np.int64))
    return torch.from_numpy(cu)


def make_topk_idx(seqlens: Sequence[int], num_kv_heads: int, topk: int, block_size: int, seed: int) -> torch.Tensor:
    """Causal block ids, ``[Hk, N, T]`` int32.  Always contains block 0 and the token's own
    block; the remaining slots are a uniform sample of earlier blocks; ascending; -1 tail."""
    rng = np.random.Generator(np.random.PCG64(seed))
    N = int(sum(seqlens))
    out = np.full((num_kv_heads, N, topk), -1, dtype=np.int32)
    start = 0
    for L in seqlens:
        nb = (L + block_size - 1) // block_size
        for b in range(nb):
            t0 = start + b * block_size
            t1 = start + min(L, (b + 1) * block_size)
            n = t1 - t0
            forced = [0] if b == 0 else [0, b]
            forced = forced[:topk]
            if topk == 1:
                forced = [b]
            rem = topk - len(forced)
            cand = b - 1  # ids 1..b-1
            tile = np.full((num_kv_heads, n, topk), np.iinfo(np.int32).max, dtype=np.int32)
            for i, f in enumerate(forced):
                tile[:, :, i] = f
            take = min(rem, max(cand, 0))
            if take > 0:
                if cand <= rem:
                    tile[:, :, len(forced):len(forced) + cand] = np.arange(1, b, dtype=np.int32)
                else:
                    keys = rng.random((num_kv_heads, n, cand), dtype=np.float32)
                    pick = np.argpartition(keys, take - 1, axis=-1)[:, :, :take].astype(np.int32) + 1
                    tile[:, :, len(forced):len(forced) + take] = pick
            tile.sort(axis=-1)
            tile[tile == np.iinfo(np.int32).max] = -1
            out[:, t0:t1] = tile
        start += L
    return torch.from_numpy(out)


def make_qkv(
    n_tokens: int, num_q_heads: int, num_kv_heads: int, head_dim: int, seed: int, dtype=torch.bfloat16, with_do: bool = True
) -> Tuple[torch.Tensor, ...]:
    """q, k, v (and dO) ~ N(0,1), drawn in fp32 on the CPU from the seed, then rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n_tokens, num_q_heads, head_dim, generator=g).to(dtype)
    k = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g).to(dtype)
    v = torch.randn(n_tokens, num_kv_heads, head_dim, generator=g).to(dtype)
    if not with_do:
        return q, k, v
    do = torch.randn(n_tokens, num_q_heads, head_dim, generator=g).to(dtype)
    return q, k, v, do
