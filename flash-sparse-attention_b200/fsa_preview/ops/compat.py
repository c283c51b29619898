"""The reference's three decode operators under their own names and argument lists
(fsa_preview/ops/__init__.py:1-9), running on the sm_100a decode kernels over PACKED tensors.

Semantics are those of the prefill path for the decoded row (the token at position
``query_start_index`` of its sequence): the reference's decode operators are not pinned by any test
and two of them disagree with its own prefill (the "local blocks" rule is evaluated at position 0,
compressed_attention_decode.py:329-355; the selected branch runs the prefill kernel with in-sequence
query index 0 and so attends key 0 only, selected_attention_decode.py:29-40).
"""
from __future__ import annotations

import math
import warnings
from typing import Optional, Tuple, Union

import torch

from fsa_preview.ops.decode import CudaDecodeOps

_OPS = CudaDecodeOps()


def _linear_compress_decode(new_tokens: torch.Tensor, compress_weight: torch.Tensor, kernel_size: int, kernel_stride: int,
                            intra_block_pe: Optional[torch.Tensor] = None, prev_total_len: int = 0,
                            token_buffer: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Incremental compressor (fsa_preview/ops/linear_compress_decode.py:14-76): ``new_tokens [1, H, d]`` extends a
    sequence of ``prev_total_len`` tokens whose last rows are ``token_buffer``; returns the ONE new compressed token
    ``[1, H, d]`` when the new length completes a window, else None."""
    if token_buffer is None:
        all_tokens, buffer_start = new_tokens, prev_total_len
    else:
        all_tokens = torch.cat([token_buffer, new_tokens], dim=0)
        buffer_start = prev_total_len - token_buffer.shape[0]
    new_len = prev_total_len + 1
    prev_max = (prev_total_len - kernel_size) // kernel_stride if prev_total_len >= kernel_size else -1
    new_max = (new_len - kernel_size) // kernel_stride if new_len >= kernel_size else -1
    if new_max <= prev_max:
        return None
    a = new_max * kernel_stride - buffer_start
    if a < 0 or a + kernel_size > all_tokens.shape[0]:
        return None
    win = all_tokens[a : a + kernel_size]                              # [ks, H, d]
    H, d = win.shape[1], win.shape[2]
    x = win.permute(1, 0, 2).reshape(H, 1, kernel_size * d)
    y = torch.bmm(x, compress_weight).transpose(0, 1)                  # [1, H, d]
    if intra_block_pe is not None:
        y = y + torch.einsum("hD,hDd->hd", intra_block_pe.reshape(H, kernel_size * d), compress_weight).unsqueeze(0)
    return y


def _positions(query_start_index: Union[int, torch.Tensor], batch: int, device) -> Tuple[torch.Tensor, int]:
    if isinstance(query_start_index, torch.Tensor):
        t = query_start_index.to(device=device, dtype=torch.int32).reshape(-1).expand(batch).contiguous()
        return t, int(t.max().item())
    return torch.full((batch,), int(query_start_index), dtype=torch.int32, device=device), int(query_start_index)


def _compressed_attention_decode(q, k, v, kernel_size: int, kernel_stride: int, block_size: int, topk: int, cu_seqlens_q,
                                 cu_seqlens_k, max_seqlen_q, max_seqlen_k, sm_scale: float = None, init_blocks: int = 1,
                                 local_blocks: int = 2, query_start_index: Union[int, torch.Tensor] = 0):
    """One query per sequence against the packed compressed K/V; returns (o ``[B, Hq, d]``, topk_idx ``[Hk, B, topk]``
    ascending, -1 padded).  ``query_start_index``: position of the query in its sequence (int, or a tensor ``[B]``)."""
    assert q.dtype in (torch.bfloat16, torch.float16) and q.dtype == k.dtype == v.dtype
    assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
    B, Hq, D = q.shape
    assert cu_seqlens_q.numel() == B + 1, "decode takes exactly one query token per sequence"
    Hk = k.shape[1]
    if sm_scale is None:
        sm_scale = 1 / math.sqrt(D)
    if max_seqlen_k is None:
        max_seqlen_k = int((cu_seqlens_k[1:] - cu_seqlens_k[:-1]).max().item())
    t, t_max = _positions(query_start_index, B, q.device)
    cmp_len = cu_seqlens_k[1:] - cu_seqlens_k[:-1]
    vis = torch.clamp((t + 1 - kernel_size) // kernel_stride + 1, min=0) * (t + 1 >= kernel_size)
    num_cmp = torch.minimum(vis.to(torch.int32), cmp_len)
    has = num_cmp > 0
    row0 = cu_seqlens_k[:-1]
    neg = torch.full_like(row0, -1)
    lo = torch.where(has, row0, neg).view(B, 1, 1).expand(B, Hk, 1).contiguous()
    hi = torch.where(has, row0 + num_cmp, neg).view(B, 1, 1).expand(B, Hk, 1).contiguous()
    chunk = 256
    nchunk = max(-(-int(max_seqlen_k) // chunk), 1)
    q = q.contiguous()
    o_part, ml, scores = _OPS.attn_partial(q, k.contiguous(), v.contiguous(), lo, hi, chunk, nchunk, sm_scale, want_scores=topk > 0)
    o, lse = _OPS.lse_merge(o_part, ml, q.dtype)
    if topk <= 0:
        warnings.warn("topk <= 0, returned topk_idx will be None")
        return o, None
    assert topk >= init_blocks + local_blocks
    ld = chunk * nchunk
    idx = _OPS.select_topk(scores, ld, ld, 0, lse, (t + 1).to(torch.int32), num_cmp, Hk, kernel_size, kernel_stride, block_size,
                           init_blocks, local_blocks, topk, t_max // block_size + 1)
    return o, idx.transpose(0, 1).contiguous()


def _topk_sparse_attention_decode(q, k, v, topk_idx, block_size: int, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                  sm_scale=None):
    """One query per sequence (the LAST token of its sequence in the packed k/v) over its selected blocks.
    ``topk_idx [Hk, B, T]``.  Returns o ``[B, Hq, d]``."""
    assert q.dtype in (torch.bfloat16, torch.float16) and q.dtype == k.dtype == v.dtype
    assert topk_idx.dtype == torch.int32 and cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
    B, Hq, D = q.shape
    assert cu_seqlens_q.numel() == B + 1, "decode takes exactly one query token per sequence"
    Hk, T = k.shape[1], topk_idx.shape[-1]
    if sm_scale is None:
        sm_scale = 1 / math.sqrt(D)
    seq_len = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).contiguous()
    lo, hi = _OPS.ranges(topk_idx.transpose(0, 1).contiguous(), seq_len, cu_seqlens_k[:-1].contiguous(), Hk, T, block_size, 0,
                         block_size, 0, 0, 2**31 - 1)
    o_part, ml, _ = _OPS.attn_partial(q.contiguous(), k.contiguous(), v.contiguous(), lo, hi, block_size, 1, sm_scale)
    o, _ = _OPS.lse_merge(o_part, ml, q.dtype)
    return o
