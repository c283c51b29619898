"""Selected (top-k block-sparse) attention: the public operator of the reference
(fsa/ops/FSA_topk_sparse_attention.py:1887-2000) on hand-written sm_100a kernels.

Same signature, same autograd behaviour (differentiable in q, k, v), same preconditions
(the reference's asserts at :1903-1906, block-size set at :926, head divisibility at :932).
The work is done by libfsa_sm100.so through its C ABI; there is no other implementation.
"""
from __future__ import annotations

import math
import os
from ctypes import byref, c_int, c_int64
from typing import Any, Optional

import torch

from fsa import _lib

__all__ = ["FSA_topk_sparse_attention", "FSATopkSparseAttention", "sel_attn_fwd", "sel_attn_bwd"]

_CHECK_STATUS = os.environ.get("FSA_CHECK_STATUS", "0") == "1"


def _rows_ok(t: torch.Tensor, need_head_packed: bool) -> bool:
    """Can the kernels read this [N, H, D] tensor in place?"""
    if t.stride(2) != 1 or t.data_ptr() % 16:
        return False
    if t.stride(0) % 8 or t.stride(1) % 8:
        return False
    if need_head_packed and t.stride(1) != t.shape[2]:
        return False
    return True


def _prep(t: torch.Tensor, need_head_packed: bool = False) -> torch.Tensor:
    return t if _rows_ok(t, need_head_packed) else t.contiguous()


def _alloc_bytes(n: int, device) -> torch.Tensor:
    return torch.empty(max(int(n), 16), dtype=torch.uint8, device=device)


def sel_attn_fwd(q, k, v, topk_idx, block_size, cu_seqlens, sm_scale, check_status: bool = False):
    """Run the forward kernels.  Returns ``(o, lse, index_ws)``; ``index_ws`` holds the
    block->entries inversion the backward reuses."""
    assert q.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
    L = _lib.lib()
    N, Hq, D = q.shape
    Hk = k.shape[1]
    T = topk_idx.shape[-1]
    B = cu_seqlens.shape[0] - 1
    q, k, v = _prep(q), _prep(k, True), _prep(v, True)
    topk_idx = topk_idx.contiguous()
    cu_seqlens = cu_seqlens.contiguous()
    dev = q.device
    nb = c_int64(0)
    _lib.check(L.fsa_sel_index_bytes(N, B, Hq, Hk, T, block_size, byref(nb)), "fsa_sel_index_bytes")
    index_ws = _alloc_bytes(nb.value, dev)
    _lib.check(L.fsa_sel_fwd_scratch_bytes(N, B, Hq, Hk, D, T, block_size, byref(nb)), "fsa_sel_fwd_scratch_bytes")
    scratch = _alloc_bytes(nb.value, dev)
    o = torch.empty((N, Hq, D), dtype=q.dtype, device=dev)
    lse = torch.empty((Hq, N), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = L.fsa_sel_fwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(topk_idx), _lib.ptr(cu_seqlens),
            N, B, Hq, Hk, D, T, block_size, _lib.DTYPE_CODE[q.dtype],
            q.stride(0), q.stride(1), k.stride(0), v.stride(0), float(sm_scale),
            _lib.ptr(o), o.stride(0), o.stride(1), _lib.ptr(lse),
            _lib.ptr(index_ws), index_ws.numel(), _lib.ptr(scratch), scratch.numel(), _lib.current_stream(dev),
        )
        _lib.check(rc, "fsa_sel_fwd")
        if check_status or _CHECK_STATUS:
            st = c_int(0)
            _lib.check(L.fsa_read_status(_lib.ptr(index_ws), _lib.current_stream(dev), byref(st)), "fsa_sel_fwd status")
    return o, lse, index_ws


def sel_attn_bwd(q, k, v, o, lse, do, topk_idx, block_size, cu_seqlens, sm_scale, index_ws, check_status: bool = False):
    """Run the backward kernels.  Returns ``(dq, dk, dv)``."""
    L = _lib.lib()
    N, Hq, D = q.shape
    Hk = k.shape[1]
    T = topk_idx.shape[-1]
    B = cu_seqlens.shape[0] - 1
    q, k, v, o, do = _prep(q), _prep(k, True), _prep(v, True), _prep(o), _prep(do)
    topk_idx = topk_idx.contiguous()
    dev = q.device
    nb = c_int64(0)
    _lib.check(L.fsa_sel_bwd_scratch_bytes(N, B, Hq, Hk, D, T, block_size, byref(nb)), "fsa_sel_bwd_scratch_bytes")
    scratch = _alloc_bytes(nb.value, dev)
    dq = torch.empty((N, Hq, D), dtype=q.dtype, device=dev)
    dk = torch.empty((N, Hk, D), dtype=q.dtype, device=dev)
    dv = torch.empty((N, Hk, D), dtype=q.dtype, device=dev)
    with torch.cuda.device(dev):
        rc = L.fsa_sel_bwd(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(do),
            _lib.ptr(topk_idx), _lib.ptr(cu_seqlens), N, B, Hq, Hk, D, T, block_size, _lib.DTYPE_CODE[q.dtype],
            q.stride(0), q.stride(1), k.stride(0), v.stride(0), o.stride(0), o.stride(1), do.stride(0), do.stride(1),
            float(sm_scale), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
            _lib.ptr(index_ws), index_ws.numel(), _lib.ptr(scratch), scratch.numel(), _lib.current_stream(dev),
        )
        _lib.check(rc, "fsa_sel_bwd")
        if check_status or _CHECK_STATUS:
            st = c_int(0)
            _lib.check(L.fsa_read_status(_lib.ptr(index_ws), _lib.current_stream(dev), byref(st)), "fsa_sel_bwd status")
    return dq, dk, dv


class FSATopkSparseAttention(torch.autograd.Function):
    """Mirror of the reference Function (fsa/ops/FSA_topk_sparse_attention.py:1887-1961): same
    forward arguments, backward returns ``dq, dk, dv`` and ``None`` for everything else."""

    @staticmethod
    def forward(ctx, q, k, v, topk_idx, block_size, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, sm_scale=None):
        assert q.dtype == torch.bfloat16 or q.dtype == torch.float16
        assert q.dtype == k.dtype and k.dtype == v.dtype
        assert topk_idx.dtype == torch.int32
        assert cu_seqlens_q.dtype == torch.int32 and cu_seqlens_k.dtype == torch.int32
        assert block_size in {32, 64, 128, 256}
        assert q.shape[1] % k.shape[1] == 0
        assert topk_idx.shape[0] == k.shape[1] and topk_idx.shape[1] == q.shape[0]
        if sm_scale is None:
            sm_scale = 1 / math.sqrt(q.shape[-1])
        o, lse, index_ws = sel_attn_fwd(q, k, v, topk_idx, block_size, cu_seqlens_q, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens_q, cu_seqlens_k, topk_idx, index_ws)
        ctx.sm_scale = sm_scale
        ctx.max_seqlen_q = max_seqlen_q
        ctx.max_seqlen_k = max_seqlen_k
        ctx.block_size = block_size
        return o

    @staticmethod
    def backward(ctx, do: torch.Tensor, *args) -> Any:
        q, k, v, o, lse, cu_seqlens_q, cu_seqlens_k, topk_idx, index_ws = ctx.saved_tensors
        dq, dk, dv = sel_attn_bwd(q, k, v, o, lse, do, topk_idx, ctx.block_size, cu_seqlens_q, ctx.sm_scale, index_ws)
        return dq, dk, dv, None, None, None, None, None, None, None, None


def FSA_topk_sparse_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    topk_idx: torch.Tensor,
    block_size: int,
    cu_seqlens: torch.Tensor,
    softmax_scale: Optional[float] = None,
) -> torch.Tensor:
    """Top-k sparse attention, varlen.

    Args:
        q: ``[total_len, num_q_heads, head_dim]`` bf16/fp16
        k, v: ``[total_len, num_kv_heads, head_dim]``
        topk_idx: ``[num_kv_heads, total_len, topk]`` int32, -1 means padding
        block_size: key/value block size (32, 64, 128 or 256)
        cu_seqlens: ``[batch_size + 1]`` int32
        softmax_scale: defaults to ``1/sqrt(head_dim)``
    Returns:
        attention output ``[total_len, num_q_heads, head_dim]``
    """
    # the reference computes max_seqlen with a host sync (:1986); the kernels here do not need it
    return FSATopkSparseAttention.apply(q, k, v, topk_idx, block_size, cu_seqlens, cu_seqlens, None, None, softmax_scale)
