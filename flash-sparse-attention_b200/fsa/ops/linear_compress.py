"""K/V compression by a strided linear projection, with the reference's interface
(nsa_ref/ops/linear_compress.py:295-502):

    y[c, h, :] = sum_{k < kernel_size} x[c * stride + k, h, :] @ W[h, k*d:(k+1)*d, :]      (+ pe bias for keys)
    compressed length = floor((L - kernel_size) / stride) + 1, or 0 when L < kernel_size   (:334-337)

This is a plain GEMM per head over overlapping windows, so it is laid out as one (the windows
are unfolded once, then a batched library GEMM): no hand-written kernel, no fp32 atomics in the
backward (the reference's backward uses tl.atomic_add, :275, :292, and is therefore not
bit-reproducible).  Everything stays on the device; the only host value needed is the list of
sequence lengths, which the caller may pass to avoid a sync.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch


def compressed_seqlens(seqlens: Sequence[int], kernel_size: int, kernel_stride: int):
    return [(L - kernel_size) // kernel_stride + 1 if L >= kernel_size else 0 for L in seqlens]


def linear_compress(
    x: torch.Tensor,
    w: torch.Tensor,
    cu_seqlens: torch.Tensor,
    kernel_size: int,
    kernel_stride: int,
    pe: Optional[torch.Tensor] = None,
    seqlens: Optional[Sequence[int]] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
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
    outs = []
    start = 0
    for L, n in zip(seqlens, ylens):
        if n > 0:
            xs = x[start : start + L]                                   # [L, H, d]
            win = xs.unfold(0, kernel_size, kernel_stride)             # [n, H, d, ks] (view; autograd folds it back)
            a = win.permute(1, 0, 3, 2).reshape(H, n, kernel_size * d)  # [H, n, ks*d]
            outs.append(torch.bmm(a, w).transpose(0, 1))              # [n, H, d]
        start += L
    y = torch.cat(outs, 0) if outs else x.new_zeros((0, H, d))
    if pe is not None:
        assert pe.dtype == x.dtype and pe.device == x.device
        bias = torch.einsum("hD,hDd->hd", pe.reshape(H, kernel_size * d), w)
        y = y + bias.unsqueeze(0)
    return y, y_cu
