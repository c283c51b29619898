"""NSA decode layer (projections, RoPE, three branches, gate mix, output projection) with the reference's
constructor and forward signature (fsa_preview/module/fsa_decode.py:12-199), plus a stateful batched ``step``.

The decoded token sits at position L-1 of its sequence and is rotated there (what the prefill layer does for that
row, fsa/module/fsa.py:106-130); the reference rotates it at position 0 (fsa_decode.py:135 with cu_seqlens_q = [0, 1]).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from fsa import _lib
from fsa.module.rope import RopeConfig, RotaryEmbedding
from fsa.ops.gate import gate_mix
from fsa.ops.linear_compress import compressed_seqlens, linear_compress
from fsa_preview.cache import DecodeCache
from fsa_preview.ops.compat import _linear_compress_decode
from fsa_preview.ops.decode import Shard, nsa_decode_attention, nsa_decode_mixed


class FlashSparseAttentionDecode(torch.nn.Module):
    def __init__(self, hidden_size: int, num_q_heads: int, num_kv_heads: int, head_dim: int, kernel_size: int, kernel_stride: int,
                 block_size: int, topk: int, init_blocks: int, local_blocks: int, window_size: int, rope_config: RopeConfig):
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
        self.rope_config = rope_config
        self.proj_q = torch.nn.Linear(hidden_size, num_q_heads * head_dim, bias=False)
        self.proj_k = torch.nn.Linear(hidden_size, num_kv_heads * head_dim, bias=False)
        self.proj_v = torch.nn.Linear(hidden_size, num_kv_heads * head_dim, bias=False)
        self.proj_o = torch.nn.Linear(num_q_heads * head_dim, hidden_size, bias=False)
        self.compress_key = torch.nn.Parameter(torch.zeros(num_kv_heads, head_dim * kernel_size, head_dim))
        self.compress_value = torch.nn.Parameter(torch.zeros(num_kv_heads, head_dim * kernel_size, head_dim))
        self.intra_block_pe = torch.nn.Parameter(torch.zeros(num_kv_heads, kernel_size, head_dim))
        self.gate = torch.nn.Sequential(torch.nn.Linear(hidden_size, 3, bias=False), torch.nn.Sigmoid())
        self.rope = RotaryEmbedding(self.rope_config)
        self.last_topk_idx = None

    def _nsa(self):
        return dict(kernel_size=self.kernel_size, kernel_stride=self.kernel_stride, block_size=self.block_size, topk=self.topk,
                    init_blocks=self.init_blocks, local_blocks=self.local_blocks, window_size=self.window_size)

    def rope_at(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotate row b of ``x [B, H, d]`` at ``positions[b]``: the rows are handed to the rotation kernel as one
        sequence whose cos / sin table row b holds the angles of positions[b]."""
        cos, sin = self.rope.generate_cos_sin(x, positions)
        B, H, D = x.shape
        x = x.contiguous()
        out = torch.empty_like(x)
        cu = torch.tensor([0, B], dtype=torch.int32, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.lib().fsa_rope(_lib.ptr(x), x.stride(0), x.stride(1), _lib.ptr(cos.contiguous()), _lib.ptr(sin.contiguous()),
                                     _lib.ptr(cu), 1, B, H, D, _lib.DTYPE_CODE[x.dtype], 0, _lib.ptr(out), _lib.current_stream(x.device))
        _lib.check(rc, "fsa_rope")
        return out

    # ------------------------------------------------------------------ stateful path
    def new_cache(self, batch: int, max_len: int, shard: Optional[Shard] = None, dtype=torch.bfloat16, device="cuda") -> DecodeCache:
        return DecodeCache(batch, max_len, self.num_kv_heads, self.head_dim, self.kernel_size, self.kernel_stride, dtype, device, shard)

    @torch.no_grad()
    def prefill_cache(self, cache: DecodeCache, x: torch.Tensor, cu_seqlens: torch.Tensor, seqlens: Optional[Sequence[int]] = None):
        """Fill ``cache`` from the prompt hidden states ``x [total, hidden]`` (projections, compression, rotation)."""
        if seqlens is None:
            seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
        k = self.proj_k(x).view(-1, self.num_kv_heads, self.head_dim)
        v = self.proj_v(x).view(-1, self.num_kv_heads, self.head_dim)
        ck, ccu = linear_compress(k, self.compress_key, cu_seqlens, self.kernel_size, self.kernel_stride, self.intra_block_pe, seqlens)
        cv, _ = linear_compress(v, self.compress_value, cu_seqlens, self.kernel_size, self.kernel_stride, None, seqlens)
        clens = compressed_seqlens(seqlens, self.kernel_size, self.kernel_stride)
        ck = self.rope(ck, ccu, start=0, stride=self.kernel_stride, max_seqlen=max(clens) if clens else 0)
        k_rot = self.rope(k, cu_seqlens, max_seqlen=max(seqlens))
        cache.load(k, k_rot, v, ck, cv, seqlens, clens)

    @torch.no_grad()
    def step(self, x: torch.Tensor, cache: DecodeCache) -> torch.Tensor:
        """``x [B, hidden]``: one new token per sequence -> ``[B, hidden]``; appends to ``cache``."""
        B = x.shape[0]
        pos = cache.seq_len.clone()                                   # position of the new token
        q = self.proj_q(x).view(B, self.num_q_heads, self.head_dim)
        k_new = self.proj_k(x).view(B, self.num_kv_heads, self.head_dim)
        v_new = self.proj_v(x).view(B, self.num_kv_heads, self.head_dim)
        q = self.rope_at(q, pos)
        cache.append(k_new, self.rope_at(k_new, pos), v_new, self.compress_key, self.compress_value, self.intra_block_pe, self.rope_at)
        gate = self.gate(x)
        if cache.shard.world == 1:
            mixed, idx = nsa_decode_mixed(q, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                          cache.cmp_row0, gate, max_len=cache.max_len, **self._nsa())
            self.last_topk_idx = idx
            return self.proj_o(mixed.flatten(1))
        oc, os_, ow, *_, idx = nsa_decode_attention(q, cache.k, cache.v, cache.cmp_k, cache.cmp_v, cache.seq_len, cache.seq_row0,
                                                    cache.cmp_row0, max_len=cache.max_len, shard=cache.shard, **self._nsa())
        self.last_topk_idx = idx
        return self.proj_o(gate_mix(gate, oc, os_.contiguous(), ow.contiguous()).flatten(1))

    # ------------------------------------------------------------------ reference signature (one sequence, stateless)
    @torch.no_grad()
    def forward(self, x, cu_seqlens_q, cu_seqlens_k, k_cache=None, v_cache=None, cmp_k_cache=None, cmp_v_cache=None):
        """``x [1, hidden]``; ``k_cache / v_cache [L-1, Hk, d]`` and the compressed caches are UN-rotated, as in the
        reference, and the whole K is rotated again on every call (use ``step`` to avoid that)."""
        assert x.dtype == torch.bfloat16 or x.dtype == torch.float16
        assert x.shape[-1] == self.hidden_size
        assert cu_seqlens_k.numel() == 2, "the stateless signature handles one sequence (as the reference); use step() for batches"
        q = self.proj_q(x).view(-1, self.num_q_heads, self.head_dim)
        k_new = self.proj_k(x).view(-1, self.num_kv_heads, self.head_dim)
        v_new = self.proj_v(x).view(-1, self.num_kv_heads, self.head_dim)
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
        dev = x.device
        C = cmp_k.shape[0]
        if C == 0:
            cmp_k = cmp_v = k.new_zeros((1, self.num_kv_heads, self.head_dim))
        else:
            cmp_k = self.rope(cmp_k, torch.tensor([0, C], dtype=torch.int32, device=dev), start=0, stride=self.kernel_stride, max_seqlen=C)
        q = self.rope_at(q, torch.tensor([L - 1], dtype=torch.int32, device=dev))
        k = self.rope(k, torch.tensor([0, L], dtype=torch.int32, device=dev), max_seqlen=L)
        one = torch.tensor([L], dtype=torch.int32, device=dev)
        zero = torch.zeros(1, dtype=torch.int32, device=dev)
        oc, os_, ow, *_, idx = nsa_decode_attention(q, k, v.contiguous(), cmp_k.contiguous(), cmp_v.contiguous(), one, zero, zero,
                                                    max_len=L, **self._nsa())
        self.last_topk_idx = idx
        gate = self.gate(x)
        return self.proj_o(gate_mix(gate, oc, os_.contiguous(), ow.contiguous()).flatten(1))
