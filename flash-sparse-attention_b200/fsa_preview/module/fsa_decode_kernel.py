"""NSA decode step without projections and RoPE, with the reference's constructor and forward signature
(fsa_preview/module/fsa_decode_kernel.py:10-176), plus a stateful batched ``step`` on a pre-allocated cache."""
from __future__ import annotations

from typing import Optional

import torch

from fsa.ops.gate import gate_mix
from fsa_preview.cache import DecodeCache
from fsa_preview.ops.compat import _linear_compress_decode
from fsa_preview.ops.decode import Shard, nsa_decode_attention, nsa_decode_mixed


class FlashSparseAttentionDecodeKernel(torch.nn.Module):
    def __init__(self, hidden_size: int, num_q_heads: int, num_kv_heads: int, head_dim: int, kernel_size: int, kernel_stride: int,
                 block_size: int, topk: int, init_blocks: int, local_blocks: int, window_size: int):
        super().__init__()
        self.hidden_size = hidden_size
        self.num_q_heads = num_q_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.kernel_size = kernel_size
        self.kernel_stride = kernel_stride
        self.block_size = block_size
        self.topk = topk
        self.init_blocks = init_blocks
        self.local_blocks = local_blocks
        self.window_size = window_size
        self.compress_key = torch.nn.Parameter(torch.zeros(num_kv_heads, head_dim * kernel_size, head_dim))
        self.compress_value = torch.nn.Parameter(torch.zeros(num_kv_heads, head_dim * kernel_size, head_dim))
        self.intra_block_pe = torch.nn.Parameter(torch.zeros(num_kv_heads, kernel_size, head_dim))
        self.gate = torch.nn.Sequential(torch.nn.Linear(hidden_size, 3, bias=False), torch.nn.Sigmoid())
        self.last_topk_idx = None

    def _nsa(self):
        return dict(kernel_size=self.kernel_size, kernel_stride=self.kernel_stride, block_size=self.block_size, topk=self.topk,
                    init_blocks=self.init_blocks, local_blocks=self.local_blocks, window_size=self.window_size)

    def new_cache(self, batch: int, max_len: int, shard: Optional[Shard] = None, dtype=torch.bfloat16, device="cuda") -> DecodeCache:
        return DecodeCache(batch, max_len, self.num_kv_heads, self.head_dim, self.kernel_size, self.kernel_stride, dtype, device, shard)

    @torch.no_grad()
    def step(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, cache: DecodeCache) -> torch.Tensor:
        """One token per sequence: ``q [B, Hq, d]``, ``k_new / v_new [B, Hk, d]`` -> ``[B, Hq*d]``; appends to ``cache``."""
        cache.append(k_new, k_new, v_new, self.compress_key, self.compress_value, self.intra_block_pe, None)
        q = q.contiguous()
        gate = self.gate(q.view(q.shape[0], -1))
        if cache.shard.world == 1:
            mixed, idx = nsa_decode_mixed(q, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                          cache.cmp_row0, gate, max_len=cache.max_len, **self._nsa())
            self.last_topk_idx = idx
            return mixed.flatten(1)
        oc, os_, ow, *_, idx = nsa_decode_attention(q, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                                    cache.cmp_row0, max_len=cache.max_len, shard=cache.shard, **self._nsa())
        self.last_topk_idx = idx
        return gate_mix(gate, oc, os_.contiguous(), ow.contiguous()).flatten(1)

    @torch.no_grad()
    def forward(self, q, k_new, v_new, cu_seqlens_q, cu_seqlens_k, k_cache=None, v_cache=None, cmp_k_cache=None, cmp_v_cache=None):
        """Reference signature, one sequence: ``q [1, Hq, d]``; ``k_cache / v_cache [L-1, Hk, d]`` and the compressed
        caches are re-concatenated on every call as the reference does (use ``step`` to avoid that)."""
        assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
        assert cu_seqlens_k.numel() == 2, "the stateless signature handles one sequence (as the reference); use step() for batches"
        q = q.view(1, self.num_q_heads, self.head_dim)
        k = torch.cat([k_cache, k_new], dim=0)
        v = torch.cat([v_cache, v_new], dim=0)
        L = k.shape[0]
        nbuf = min(self.kernel_size - 1, k_cache.shape[0])
        ck = _linear_compress_decode(k_new, self.compress_key, self.kernel_size, self.kernel_stride, self.intra_block_pe, L - 1,
                                     k_cache[L - 1 - nbuf :] if nbuf else None)
        cv = _linear_compress_decode(v_new, self.compress_value, self.kernel_size, self.kernel_stride, None, L - 1,
                                     v_cache[L - 1 - nbuf :] if nbuf else None)
        cmp_k = torch.cat([cmp_k_cache, ck], 0) if ck is not None else cmp_k_cache
        cmp_v = torch.cat([cmp_v_cache, cv], 0) if cv is not None else cmp_v_cache
        if cmp_k.shape[0] == 0:
            cmp_k = cmp_v = k.new_zeros((1, self.num_kv_heads, self.head_dim))
        dev = q.device
        one = torch.tensor([L], dtype=torch.int32, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        oc, os_, ow, *_, idx = nsa_decode_attention(q.contiguous(), k, v, cmp_k.contiguous(), cmp_v.contiguous(), one, zero, zero,
                                                    max_len=L, **self._nsa())
        self.last_topk_idx = idx
        gate = self.gate(q.view(1, -1))
        return gate_mix(gate, oc, os_.contiguous(), ow.contiguous()).flatten(1)
