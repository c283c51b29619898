"""FlashSparseAttention layer with the reference's constructor, parameters and forward
(fsa/module/fsa.py:12-173): q/k/v/o projections (library GEMMs), K/V compression, RoPE,
compressed attention -> top-k block ids, selected attention, sliding-window attention, sigmoid
gate mix, output projection.  Parameter names and shapes are the reference's, so its state_dict
loads unchanged.  All attention kernels are the sm_100a ones of libfsa_sm100.so.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from fsa.module.rope import RopeConfig, RotaryEmbedding
from fsa.ops.compressed_attention import compressed_attention
from fsa.ops.FSA_topk_sparse_attention import FSA_topk_sparse_attention
from fsa.ops.gate import gate_mix, gate_proj_mix
from fsa.ops.linear_compress import compressed_seqlens, linear_compress
from fsa.ops.range_attention import sliding_window_attention

__all__ = ["FlashSparseAttention", "RopeConfig", "RotaryEmbedding"]


class FlashSparseAttention(torch.nn.Module):
    def __init__(
        self,
        hidden_size: int,
        num_q_heads: int,
        num_kv_heads: int,
        head_dim: int,
        kernel_size: int,
        kernel_stride: int,
        block_size: int,
        topk: int,
        init_blocks: int,
        local_blocks: int,
        window_size: int,
        rope_config: RopeConfig,
    ):
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

        self.proj_q = torch.nn.Linear(self.hidden_size, self.num_q_heads * self.head_dim, bias=False)
        self.proj_k = torch.nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=False)
        self.proj_v = torch.nn.Linear(self.hidden_size, self.num_kv_heads * self.head_dim, bias=False)
        self.proj_o = torch.nn.Linear(self.num_q_heads * self.head_dim, self.hidden_size, bias=False)

        self.compress_key = torch.nn.Parameter(torch.zeros(self.num_kv_heads, self.head_dim * self.kernel_size, self.head_dim))
        self.compress_value = torch.nn.Parameter(torch.zeros(self.num_kv_heads, self.head_dim * self.kernel_size, self.head_dim))
        self.intra_block_pe = torch.nn.Parameter(torch.zeros(self.num_kv_heads, self.kernel_size, self.head_dim))

        self.gate = torch.nn.Sequential(torch.nn.Linear(self.hidden_size, 3, bias=False), torch.nn.Sigmoid())
        self.rope = RotaryEmbedding(self.rope_config)
        self.last_topk_idx = None
        self.init_params()

    def init_params(self):
        for p in self.parameters():
            torch.nn.init.xavier_uniform_(p)

    def forward(self, x: torch.Tensor, cu_seqlens: torch.Tensor, seqlens: Optional[Sequence[int]] = None):
        """``x [total_len, hidden_size]`` bf16/fp16, ``cu_seqlens [batch + 1]``.  ``seqlens`` (host list of the
        sequence lengths) is optional: passing it removes the one host sync this forward otherwise makes."""
        assert x.dtype == torch.bfloat16 or x.dtype == torch.float16
        assert x.shape[-1] == self.hidden_size
        cu_seqlens = cu_seqlens.to(torch.int32)
        if seqlens is None:
            seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
        max_len = max(seqlens) if len(seqlens) else 0
        cmp_lens = compressed_seqlens(seqlens, self.kernel_size, self.kernel_stride)
        max_cmp = max(cmp_lens) if len(cmp_lens) else 0

        q = self.proj_q(x).view(-1, self.num_q_heads, self.head_dim)
        k = self.proj_k(x).view(-1, self.num_kv_heads, self.head_dim)
        v = self.proj_v(x).view(-1, self.num_kv_heads, self.head_dim)

        compressed_k, compressed_cu_seqlens = linear_compress(
            k, self.compress_key, cu_seqlens, self.kernel_size, self.kernel_stride, self.intra_block_pe, seqlens=seqlens)
        compressed_v, _ = linear_compress(v, self.compress_value, cu_seqlens, self.kernel_size, self.kernel_stride, None, seqlens=seqlens)

        q = self.rope(q, cu_seqlens, max_seqlen=max_len)
        compressed_k = self.rope(compressed_k, compressed_cu_seqlens, start=0, stride=self.kernel_stride, max_seqlen=max_cmp)

        compressed_attn_output, topk_idx = compressed_attention(
            q, compressed_k, compressed_v, self.kernel_size, self.kernel_stride, self.block_size, self.topk,
            cu_seqlens, compressed_cu_seqlens, max_len, max_cmp, None, self.init_blocks, self.local_blocks,
            parallel_topk_compute=False, seqlens_q=seqlens, seqlens_k=cmp_lens)

        self.last_topk_idx = topk_idx      # kept for inspection (the ids are not differentiable)

        k = self.rope(k, cu_seqlens, max_seqlen=max_len)

        # the reference falls back to the query-outer kernel for GQA groups > 8 (:139-146); the kernels here
        # batch gathered tokens per head, so one kernel serves every group size
        sparse_attn_output = FSA_topk_sparse_attention(q, k, v, topk_idx, self.block_size, cu_seqlens, None)
        sliding_attn_output, _ = sliding_window_attention(q, k, v, cu_seqlens, self.window_size)

        # gate = sigmoid(Linear(hidden, 3)(x)) and the mix of the three branches, fused (same rounding points as the modules)
        if x.is_cuda and self.hidden_size % 8 == 0 and self.hidden_size <= 16384:
            attn_output = gate_proj_mix(x, self.gate[0].weight, compressed_attn_output, sparse_attn_output, sliding_attn_output)
        else:
            attn_output = gate_mix(self.gate(x), compressed_attn_output, sparse_attn_output, sliding_attn_output)
        attn_output = attn_output.reshape(attn_output.shape[0], -1)
        return self.proj_o(attn_output)
