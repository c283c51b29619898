"""Range attention on the sm_100a selected-attention kernels: every token attends a contiguous
range of K/V rows.  It carries the two dense NSA branches:

* the **compressed branch** (`compressed_attention_core`), replacing ``CompressedAttention``
  (nsa_ref/ops/compressed_attention.py:762-829): queries attend compressed tokens ``c`` with
  ``t_local >= c * kernel_stride + kernel_size - 1`` (:77-80);
* the **sliding-window branch** (`sliding_window_attention`), replacing
  ``flash_attn_varlen_func(q, k, v, ..., causal=True, window_size=(W, -1))`` as called by the layer
  (fsa/module/fsa.py:149-159): key ``j`` is visible iff ``t - W <= j <= t``.

Both return the output and the log-sum-exp in log2 units ``[num_q_heads, total_len]``.
"""
from __future__ import annotations

import math
from ctypes import byref, c_int, c_int64
from typing import Optional, Tuple

import torch

from fsa import _lib
from fsa.ops.FSA_topk_sparse_attention import _alloc_bytes, _prep

__all__ = ["range_attention", "compressed_attention_core", "sliding_window_attention", "compressed_limits", "window_limits"]

BLOCK = 64  # K/V rows per tile of the underlying kernels


def _sizes(N, Nk, B, Hq, Hk, D, max_blocks):
    L = _lib.lib()
    a, b, c = c_int64(0), c_int64(0), c_int64(0)
    _lib.check(L.fsa_range_attn_bytes(N, Nk, B, Hq, Hk, D, max_blocks, BLOCK, byref(a), byref(b), byref(c)), "fsa_range_attn_bytes")
    return a.value, b.value, c.value


class RangeAttention(torch.autograd.Function):
    """Forward: the query-tile-major kernel (``fsa_range_attn_fwd_dense``: accumulator in TMEM across the K/V tiles, no
    partial rows) for head sizes 64 / 128, else the block-major kernels.  Backward: the block-major kernels on a tile
    index (built in the backward when the forward did not leave one)."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, kv_lo, kv_hi, max_blocks, sm_scale):
        assert q.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
        assert q.dtype in (torch.bfloat16, torch.float16) and q.dtype == k.dtype == v.dtype
        assert cu_q.dtype == torch.int32 and cu_k.dtype == torch.int32 and kv_hi.dtype == torch.int32
        L = _lib.lib()
        N, Hq, D = q.shape
        Nk, Hk = k.shape[0], k.shape[1]
        B = cu_q.numel() - 1
        q, k, v = _prep(q), _prep(k, True), _prep(v, True)
        dev = q.device
        o = torch.empty((N, Hq, D), dtype=q.dtype, device=dev)
        lse = torch.empty((Hq, N), dtype=torch.float32, device=dev)
        dense = D in (64, 128) and Hq // Hk <= 32
        index_ws = None
        with torch.cuda.device(dev):
            if dense:
                rc = L.fsa_range_attn_fwd_dense(
                    _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(cu_q), _lib.ptr(cu_k), _lib.ptr(kv_lo), _lib.ptr(kv_hi),
                    N, Nk, B, Hq, Hk, D, _lib.DTYPE_CODE[q.dtype], q.stride(0), q.stride(1), k.stride(0), v.stride(0),
                    float(sm_scale), _lib.ptr(o), o.stride(0), o.stride(1), _lib.ptr(lse), None, _lib.current_stream(dev))
                _lib.check(rc, "fsa_range_attn_fwd_dense")
            else:
                ib, fb, _ = _sizes(N, Nk, B, Hq, Hk, D, max_blocks)
                index_ws, scratch = _alloc_bytes(ib, dev), _alloc_bytes(fb, dev)
                rc = L.fsa_range_attn_fwd(
                    _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(cu_q), _lib.ptr(cu_k), _lib.ptr(kv_lo), _lib.ptr(kv_hi),
                    N, Nk, B, Hq, Hk, D, max_blocks, BLOCK, _lib.DTYPE_CODE[q.dtype],
                    q.stride(0), q.stride(1), k.stride(0), v.stride(0), float(sm_scale),
                    _lib.ptr(o), o.stride(0), o.stride(1), _lib.ptr(lse),
                    _lib.ptr(index_ws), index_ws.numel(), _lib.ptr(scratch), scratch.numel(), _lib.current_stream(dev))
                _lib.check(rc, "fsa_range_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k, kv_lo if kv_lo is not None else torch.empty(0), kv_hi,
                              index_ws if index_ws is not None else torch.empty(0))
        ctx.has_lo = kv_lo is not None
        ctx.has_index = index_ws is not None
        ctx.max_blocks = max_blocks
        ctx.sm_scale = sm_scale
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, cu_q, cu_k, kv_lo, kv_hi, index_ws = ctx.saved_tensors
        kv_lo = kv_lo if ctx.has_lo else None
        L = _lib.lib()
        N, Hq, D = q.shape
        Nk, Hk = k.shape[0], k.shape[1]
        B = cu_q.numel() - 1
        do = _prep(do)
        dev = q.device
        ib, _, bb = _sizes(N, Nk, B, Hq, Hk, D, ctx.max_blocks)
        scratch = _alloc_bytes(bb, dev)
        if not ctx.has_index:
            index_ws = _alloc_bytes(ib, dev)
            with torch.cuda.device(dev):
                rc = L.fsa_range_attn_index(_lib.ptr(cu_q), _lib.ptr(cu_k), _lib.ptr(kv_lo), _lib.ptr(kv_hi), N, Nk, B, Hq, Hk,
                                            ctx.max_blocks, BLOCK, _lib.ptr(index_ws), index_ws.numel(), _lib.current_stream(dev))
            _lib.check(rc, "fsa_range_attn_index")
        dq = torch.empty((N, Hq, D), dtype=q.dtype, device=dev)
        dk = torch.empty((Nk, Hk, D), dtype=q.dtype, device=dev)
        dv = torch.empty((Nk, Hk, D), dtype=q.dtype, device=dev)
        with torch.cuda.device(dev):
            rc = L.fsa_range_attn_bwd(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse), _lib.ptr(do), _lib.ptr(cu_q), _lib.ptr(cu_k),
                _lib.ptr(kv_lo), _lib.ptr(kv_hi), N, Nk, B, Hq, Hk, D, ctx.max_blocks, BLOCK, _lib.DTYPE_CODE[q.dtype],
                q.stride(0), q.stride(1), k.stride(0), v.stride(0), o.stride(0), o.stride(1), do.stride(0), do.stride(1),
                float(ctx.sm_scale), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
                _lib.ptr(index_ws), index_ws.numel(), _lib.ptr(scratch), scratch.numel(), _lib.current_stream(dev))
            _lib.check(rc, "fsa_range_attn_bwd")
        return dq, dk, dv, None, None, None, None, None, None


def range_attention(q, k, v, cu_q, cu_k, kv_lo, kv_hi, max_blocks, sm_scale=None):
    """``o, lse``: token n attends K/V rows ``kv_lo[n]..kv_hi[n]`` (global rows; ``kv_lo`` may be None)."""
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    if k.shape[0] == 0:
        # no K/V row exists (e.g. every sequence is shorter than the compression window): every query sees
        # nothing, which the reference defines as o = 0, lse = -inf (nsa_ref/ops/compressed_attention.py:548-553)
        assert q.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
        lse = torch.full((q.shape[1], q.shape[0]), float("-inf"), dtype=torch.float32, device=q.device)
        return q * 0, lse
    return RangeAttention.apply(q, k, v, cu_q, cu_k, kv_lo, kv_hi, int(max_blocks), float(sm_scale))


def _token_seq_and_local(cu: torch.Tensor, n_tokens: int):
    """Per token: sequence index and position inside its sequence (device tensors, no host sync)."""
    tok = torch.arange(n_tokens, device=cu.device, dtype=torch.int32)
    seq = torch.searchsorted(cu[1:].contiguous(), tok, right=True).to(torch.int64)
    return seq, tok - cu[seq]


def compressed_limits(cu_q, cu_k, n_tokens, kernel_size, kernel_stride):
    """Highest visible compressed row per token: ``cu_k[b] + (t_local - kernel_size + 1) // kernel_stride`` or -1."""
    seq, t_local = _token_seq_and_local(cu_q, n_tokens)
    lim = torch.div(t_local - (kernel_size - 1), kernel_stride, rounding_mode="floor")
    n_cmp = (cu_k[1:] - cu_k[:-1])[seq]
    lim = torch.minimum(lim, n_cmp - 1)
    hi = torch.where(lim >= 0, cu_k[seq] + lim, torch.full_like(lim, -1))
    return hi.to(torch.int32)


def window_limits(cu, n_tokens, window):
    seq, t_local = _token_seq_and_local(cu, n_tokens)
    tok = torch.arange(n_tokens, device=cu.device, dtype=torch.int32)
    lo = torch.maximum(cu[seq], tok - window)
    return lo.to(torch.int32), tok


def compressed_attention_core(q, ck, cv, kernel_size, kernel_stride, cu_q, cu_k, max_seqlen_k: int, sm_scale=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of every query over the compressed keys/values it may see.  ``max_seqlen_k`` is the
    longest compressed sequence (a host integer the caller already has)."""
    hi = compressed_limits(cu_q, cu_k, q.shape[0], kernel_size, kernel_stride)
    max_blocks = (int(max_seqlen_k) + BLOCK - 1) // BLOCK + 1
    return range_attention(q, ck, cv, cu_q, cu_k, None, hi, max_blocks, sm_scale)


def sliding_window_attention(q, k, v, cu_seqlens, window_size: int, sm_scale: Optional[float] = None):
    lo, hi = window_limits(cu_seqlens, q.shape[0], window_size)
    max_blocks = (window_size + 1 + BLOCK - 1) // BLOCK + 1
    return range_attention(q, k, v, cu_seqlens, cu_seqlens, lo, hi, max_blocks, sm_scale)
