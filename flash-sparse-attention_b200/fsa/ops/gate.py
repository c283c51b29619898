"""Sigmoid-gate mix of the three branches (fsa/module/fsa.py:162-167) as one fused kernel each way, and the same with the
gate projection and the sigmoid inside (``gate_proj_mix``: x, the [3, hidden] weight and the three branch outputs in, the
mixed output out)."""
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


class GateProjMix(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gate, a, b, c):
        assert a.is_cuda, "the sm_100a kernels need CUDA tensors (no CPU fallback)"
        xk = x if (x.stride(-1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0) else x.contiguous()
        wk, a, b, c = w_gate.contiguous(), a.contiguous(), b.contiguous(), c.contiguous()
        N, hidden = xk.shape
        row = a[0].numel() if N else 0
        out = torch.empty_like(a)
        gate = torch.empty((N, 3), dtype=a.dtype, device=a.device)
        with torch.cuda.device(a.device):
            rc = _lib.lib().fsa_gate_proj_mix_fwd(_lib.ptr(xk), xk.stride(0), _lib.ptr(wk), _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), N, hidden, row,
                                                  _lib.DTYPE_CODE[a.dtype], _lib.ptr(out), _lib.ptr(gate), _lib.current_stream(a.device))
        _lib.check(rc, "fsa_gate_proj_mix_fwd")
        ctx.save_for_backward(xk, wk, gate, a, b, c)
        return out

    @staticmethod
    def backward(ctx, dout):
        xk, wk, gate, a, b, c = ctx.saved_tensors
        dout = dout.contiguous()
        N, hidden = xk.shape
        row = a[0].numel() if N else 0
        da, db, dc = torch.empty_like(a), torch.empty_like(b), torch.empty_like(c)
        dx = torch.empty((N, hidden), dtype=xk.dtype, device=xk.device)
        dw = torch.empty_like(wk)
        L = _lib.lib()
        scratch = torch.empty(max(int(L.fsa_gate_proj_mix_scratch_bytes(N, hidden)), 16), dtype=torch.uint8, device=xk.device)
        with torch.cuda.device(a.device):
            rc = L.fsa_gate_proj_mix_bwd(_lib.ptr(xk), xk.stride(0), _lib.ptr(wk), _lib.ptr(gate), _lib.ptr(a), _lib.ptr(b), _lib.ptr(c),
                                         _lib.ptr(dout), N, hidden, row, _lib.DTYPE_CODE[a.dtype], _lib.ptr(da), _lib.ptr(db), _lib.ptr(dc),
                                         _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(scratch), scratch.numel(), _lib.current_stream(a.device))
        _lib.check(rc, "fsa_gate_proj_mix_bwd")
        if N == 0:
            dx.zero_(); dw.zero_()
        return dx, dw, da, db, dc


def gate_proj_mix(x: torch.Tensor, w_gate: torch.Tensor, a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """``sigmoid(x @ w_gate.T)`` ([N, 3]) mixing ``a, b, c [N, H, d]``: the gate Linear, the sigmoid and the mix in one kernel."""
    return GateProjMix.apply(x, w_gate, a, b, c)
