"""Compressed-branch attention + top-k block selection with the reference's interface
(``compressed_attention``, nsa_ref/ops/compressed_attention.py:1161-1317).

The attention itself runs on the sm_100a range-attention kernels.  The selection is one fused kernel
(``fsa_select_topk_fused``: q.k^T on the tensor cores, probabilities, block scores, top-k, no score tensor in memory);
shapes outside what that kernel is compiled for take the two-step path (a batched library GEMM per sequence writing the
raw products in fp32, then ``fsa_select_topk_seq``).
"""
from __future__ import annotations

import math
import warnings
from typing import Optional, Sequence, Tuple

import torch

from fsa import _lib
from fsa.ops.range_attention import compressed_attention_core


_FUSED_TAPS = {(2, 2), (2, 4), (2, 8), (1, 4), (4, 4), (4, 8)}     # (kernel_size / stride, block_size / stride) the fused kernel is compiled for


def select_topk_blocks(q, ck, lse, kernel_size, kernel_stride, block_size, topk, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                       sm_scale, init_blocks=1, local_blocks=2, seqlens_q: Optional[Sequence[int]] = None,
                       seqlens_k: Optional[Sequence[int]] = None) -> torch.Tensor:
    """``topk_idx [Hk, N, min(topk, max_blocks)]`` int32: ascending sequence-local block ids, -1 padded."""
    L = _lib.lib()
    N, Hq, d = q.shape
    Hk = ck.shape[1]
    G = Hq // Hk
    max_blocks = math.ceil(max_seqlen_q / block_size)
    t_out = min(topk, max_blocks)
    if seqlens_q is None:
        seqlens_q = (cu_seqlens_q[1:] - cu_seqlens_q[:-1]).tolist()
    if seqlens_k is None:
        seqlens_k = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).tolist()
    out = torch.empty((Hk, N, t_out), dtype=torch.int32, device=q.device)
    lse = lse.contiguous()
    a, bsr = kernel_size // kernel_stride, block_size // kernel_stride
    fused_ok = (d in (64, 128) and t_out <= 32 and (a, bsr) in _FUSED_TAPS and kernel_size % kernel_stride == 0
                and block_size % kernel_stride == 0)
    if fused_ok:
        qf = q if (q.stride(2) == 1 and q.stride(1) == d and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0) else q.contiguous()
        kf = ck if (ck.stride(2) == 1 and ck.stride(1) == d and ck.stride(0) % 8 == 0 and ck.data_ptr() % 16 == 0) else ck.contiguous()
        with torch.cuda.device(q.device):
            rc = L.fsa_select_topk_fused(_lib.ptr(qf), qf.stride(0), _lib.ptr(kf) if kf.shape[0] else None, kf.stride(0) if kf.shape[0] else Hk * d,
                                         _lib.ptr(lse), _lib.ptr(cu_seqlens_q), _lib.ptr(cu_seqlens_k), N, kf.shape[0], cu_seqlens_q.numel() - 1,
                                         Hq, Hk, d, _lib.DTYPE_CODE[q.dtype], float(sm_scale), kernel_size, kernel_stride, block_size,
                                         init_blocks, local_blocks, max_blocks, t_out, _lib.ptr(out), None, _lib.current_stream(q.device))
        _lib.check(rc, "fsa_select_topk_fused")
        return out
    qs = ks = 0
    with torch.cuda.device(q.device):
        for Lq, Lk in zip(seqlens_q, seqlens_k):
            if Lq > 0:
                q0 = q[qs : qs + Lq, ::G].transpose(0, 1)                 # [Hk, Lq, d] first head of each group
                ld = max((Lk + 3) // 4 * 4, 4)
                if Lk > 0:
                    kk = ck[ks : ks + Lk]
                    if ld != Lk:
                        kk = torch.nn.functional.pad(kk, (0, 0, 0, 0, 0, ld - Lk))   # zero rows: the row stride stays 16-byte aligned
                    # 16-bit operands, fp32 accumulation and fp32 output on the tensor cores (the products are exact;
                    # the reference's score kernel does the same with tl.dot)
                    qk = torch.bmm(q0, kk.permute(1, 2, 0), out_dtype=torch.float32)   # [Hk, Lq, ld]
                else:
                    qk = torch.zeros((Hk, Lq, ld), dtype=torch.float32, device=q.device)
                rc = L.fsa_select_topk_seq(_lib.ptr(qk), ld, _lib.ptr(lse), N, qs, Lq, Lk, Hk, G, float(sm_scale), kernel_size,
                                           kernel_stride, block_size, init_blocks, local_blocks, max_blocks, t_out, _lib.ptr(out),
                                           _lib.current_stream(q.device))
                _lib.check(rc, "fsa_select_topk_seq")
            qs += Lq
            ks += Lk
    return out


def compressed_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    kernel_size: int,
    kernel_stride: int,
    block_size: int,
    topk: int,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    sm_scale: float = None,
    init_blocks: int = 1,
    local_blocks: int = 2,
    parallel_topk_compute="auto",
    seqlens_q: Optional[Sequence[int]] = None,
    seqlens_k: Optional[Sequence[int]] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Attention between queries and compressed keys/values, and the top-k block ids for the
    selected branch.  Same arguments and return contract as the reference; ``parallel_topk_compute``
    is accepted and ignored (there is one selection kernel)."""
    if max_seqlen_q is None:
        max_seqlen_q = int((cu_seqlens_q[1:] - cu_seqlens_q[:-1]).max().item())
    if max_seqlen_k is None:
        max_seqlen_k = int((cu_seqlens_k[1:] - cu_seqlens_k[:-1]).max().item())
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    o, lse = compressed_attention_core(q, k, v, kernel_size, kernel_stride, cu_seqlens_q, cu_seqlens_k, max_seqlen_k, sm_scale)
    if topk <= 0:
        warnings.warn("topk <= 0, returned topk_idx will be None")
        return o, None
    assert topk >= init_blocks + local_blocks
    with torch.no_grad():
        topk_idx = select_topk_blocks(q.detach(), k.detach(), lse, kernel_size, kernel_stride, block_size, topk, cu_seqlens_q,
                                      cu_seqlens_k, max_seqlen_q, sm_scale, init_blocks, local_blocks, seqlens_q, seqlens_k)
    return o, topk_idx
