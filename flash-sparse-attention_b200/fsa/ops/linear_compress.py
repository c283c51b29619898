"""K/V compression by a strided linear projection, with the reference's interface
(nsa_ref/ops/linear_compress.py:295-502):

    y[c, h, :] = sum_{k < kernel_size} x[c * stride + k, h, :] @ W[h, k*d:(k+1)*d, :]      (+ pe bias for keys)
    compressed length = floor((L - kernel_size) / stride) + 1, or 0 when L < kernel_size   (:334-337)

Forward: ``fsa_linear_compress_fwd``, a tcgen05 GEMM per (128 windows, head) that reads the overlapping token windows in
place through a strided TMA map and adds the bias in its epilogue (head_dim 64 / 128).  Backward:
``fsa_linear_compress_bwd``, two tcgen05 GEMM kernels (dx per token phase, dW with the window index as the reduction)
that write every gradient row once -- no fp32 atomics (the reference's backward uses tl.atomic_add, :275, :292, and is
therefore not bit-reproducible).  Other head sizes use a batched library GEMM over the unfolded windows, differentiated
by autograd.  Everything stays on the device; the only host value needed is the list of sequence lengths, which
the caller may pass to avoid a sync.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np
import torch

from fsa import _lib


def compressed_seqlens(seqlens: Sequence[int], kernel_size: int, kernel_stride: int):
    return [(L - kernel_size) // kernel_stride + 1 if L >= kernel_size else 0 for L in seqlens]


def _compress_gemm(x, w, seqlens, ylens, kernel_size, kernel_stride):
    """The product as a batched library GEMM over unfolded windows (differentiable)."""
    H, d = x.shape[1], x.shape[2]
    outs, start = [], 0
    for L, n in zip(seqlens, ylens):
        if n > 0:
            xs = x[start : start + L]                                   # [L, H, d]
            win = xs.unfold(0, kernel_size, kernel_stride)             # [n, H, d, ks] (view; autograd folds it back)
            a = win.permute(1, 0, 3, 2).reshape(H, n, kernel_size * d)  # [H, n, ks*d]
            outs.append(torch.bmm(a, w).transpose(0, 1))              # [n, H, d]
        start += L
    return torch.cat(outs, 0) if outs else x.new_zeros((0, H, d))


class _LinearCompress(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, cu_seqlens, seqlens, ylens, kernel_size, kernel_stride):
        assert x.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
        N, H, d = x.shape
        xk = x if (x.stride(2) == 1 and x.stride(1) == d and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0) else x.contiguous()
        wk = w.contiguous()
        y = torch.empty((sum(ylens), H, d), dtype=x.dtype, device=x.device)
        if y.numel():
            lens = np.asarray(seqlens, dtype=np.int32)
            bk = bias.contiguous() if bias is not None else None
            with torch.cuda.device(x.device):
                rc = _lib.lib().fsa_linear_compress_fwd(_lib.ptr(xk), xk.stride(0), _lib.ptr(wk), _lib.ptr(bk), lens.ctypes.data, len(seqlens),
                                                        H, d, kernel_size, kernel_stride, _lib.DTYPE_CODE[x.dtype], _lib.ptr(y), None,
                                                        _lib.current_stream(x.device))
            _lib.check(rc, "fsa_linear_compress_fwd")
        ctx.save_for_backward(xk, wk, cu_seqlens)
        ctx.meta = (list(seqlens), list(ylens), kernel_size, kernel_stride, bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        xk, wk, cu = ctx.saved_tensors
        seqlens, ylens, ks, st, has_bias = ctx.meta
        N, H, d = xk.shape
        dx = torch.empty((N, H, d), dtype=xk.dtype, device=xk.device) if ctx.needs_input_grad[0] else None
        dw = torch.empty_like(wk) if ctx.needs_input_grad[1] else None
        dyk = dy.contiguous()
        if dx is not None or dw is not None:
            lens = np.asarray(seqlens, dtype=np.int32)
            with torch.cuda.device(xk.device):
                rc = _lib.lib().fsa_linear_compress_bwd(_lib.ptr(xk), xk.stride(0), _lib.ptr(wk), _lib.ptr(dyk) if dyk.numel() else None,
                                                        _lib.ptr(cu), lens.ctypes.data, len(seqlens), H, d, ks, st,
                                                        _lib.DTYPE_CODE[xk.dtype], _lib.ptr(dx), _lib.ptr(dw), None,
                                                        _lib.current_stream(xk.device))
            _lib.check(rc, "fsa_linear_compress_bwd")
        dbias = dy.sum(0).to(dy.dtype) if has_bias else None
        return dx, dw, dbias, None, None, None, None, None


def linear_compress_gemm(x, w, cu_seqlens, kernel_size, kernel_stride, pe=None, seqlens=None):
    """The same operator written as a batched library GEMM over unfolded windows, on whatever device the tensors live:
    the formulation the backward differentiates, also used by host-side checks of the incremental (decode) compressor.
    Not the training / prefill path: that is ``linear_compress``."""
    H, d = x.shape[1], x.shape[2]
    if seqlens is None:
        seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    ylens = compressed_seqlens(seqlens, kernel_size, kernel_stride)
    y_cu = torch.zeros(len(seqlens) + 1, dtype=torch.int32)
    y_cu[1:] = torch.tensor(ylens, dtype=torch.int32).cumsum(0)
    y = _compress_gemm(x, w, seqlens, ylens, kernel_size, kernel_stride)
    if pe is not None:
        y = y + torch.einsum("hD,hDd->hd", pe.reshape(H, kernel_size * d), w).unsqueeze(0)
    return y, y_cu.to(x.device)


def linear_compress(
    x: torch.Tensor,
    w: torch.Tensor,
    cu_seqlens: torch.Tensor,
    kernel_size: int,
    kernel_stride: int,
    pe: Optional[torch.Tensor] = None,
    seqlens: Optional[Sequence[int]] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    assert x.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
    assert x.dtype in (torch.float16, torch.bfloat16) and x.dtype == w.dtype
    assert cu_seqlens.dtype == torch.int32
    total_len, H, d = x.shape
    assert w.shape == (H, kernel_size * d, d)
    assert kernel_size % kernel_stride == 0 and kernel_size in {16, 32, 64, 128} and d % 8 == 0
    if seqlens is None:
        seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).tolist()
    ylens = compressed_seqlens(seqlens, kernel_size, kernel_stride)
    y_cu = torch.zeros(len(seqlens) + 1, dtype=torch.int32)
    y_cu[1:] = torch.tensor(ylens, dtype=torch.int32).cumsum(0)
    y_cu = y_cu.to(x.device)
    bias = None
    if pe is not None:
        assert pe.dtype == x.dtype and pe.device == x.device
        # bias[h, :] = sum_D pe[h, D] w[h, D, :] as a broadcast product and a column sum (fp32, rounded once): the batched
        # GEMM with one row that einsum would launch, and the rank-1 GEMMs of its backward, are far slower than this
        bias = (pe.reshape(H, kernel_size * d, 1).float() * w.float()).sum(1).to(x.dtype)
    if d in (64, 128):
        y = _LinearCompress.apply(x, w, bias, cu_seqlens, seqlens, ylens, kernel_size, kernel_stride)
    else:
        y = _compress_gemm(x, w, seqlens, ylens, kernel_size, kernel_stride)
        if bias is not None:
            y = y + bias.unsqueeze(0)
    return y, y_cu
