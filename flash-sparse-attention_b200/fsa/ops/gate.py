"""Sigmoid-gate mix of the three branches (fsa/module/fsa.py:162-167) as one fused kernel each way."""
from __future__ import annotations

import torch

from fsa import _lib


class GateMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, a, b, c):
        assert a.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
        gate, a, b, c = gate.contiguous(), a.contiguous(), b.contiguous(), c.contiguous()
        N = a.shape[0]
        row = a[0].numel() if N else 0
        out = torch.empty_like(a)
        with torch.cuda.device(a.device):
            rc = _lib.lib().fsa_gate_mix_fwd(_lib.ptr(gate), _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), N, row, _lib.DTYPE_CODE[a.dtype],
                                             _lib.ptr(out), _lib.current_stream(a.device))
        _lib.check(rc, "fsa_gate_mix_fwd")
        ctx.save_for_backward(gate, a, b, c)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, a, b, c = ctx.saved_tensors
        dout = dout.contiguous()
        N = a.shape[0]
        row = a[0].numel() if N else 0
        da, db, dc = torch.empty_like(a), torch.empty_like(b), torch.empty_like(c)
        dg = torch.empty((N, 3), dtype=torch.float32, device=a.device)
        with torch.cuda.device(a.device):
            rc = _lib.lib().fsa_gate_mix_bwd(_lib.ptr(gate), _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(dout), N, row,
                                             _lib.DTYPE_CODE[a.dtype], _lib.ptr(da), _lib.ptr(db), _lib.ptr(dc), _lib.ptr(dg),
                                             _lib.current_stream(a.device))
        _lib.check(rc, "fsa_gate_mix_bwd")
        return dg.to(gate.dtype), da, db, dc


def gate_mix(gate: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``gate [N, 3]`` (after the sigmoid); ``a, b, c [N, H, d]``; returns ``g0 a + g1 b + g2 c``."""
    return GateMix.apply(gate, a, b, c)
